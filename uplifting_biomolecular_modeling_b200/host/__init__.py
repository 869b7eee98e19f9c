"""Host-side work off the critical path: content-addressed memo of expensive builds, ordered prefetch of the
next item, bulk device-to-host transfer with background writing, cold start without redundant initialisation."""
