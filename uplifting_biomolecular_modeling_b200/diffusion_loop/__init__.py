"""Helpers around a sampling loop: RNG discipline for captured / batched steps, the refuse-to-patch rule over a
stock function, and the census of host synchronisations a step makes."""
