"""Mode vocabulary and resolution.

A kit declares a :class:`ModeTable` (it must contain ``off``); the mode of a run is resolved with
precedence command line > environment variable > the kit's default, and an unknown word is an
error that names the known ones (reference: common/opt_core/opt_core/modes.py:57,93,103).
"""
from __future__ import annotations

import os
import shlex
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

MODE_WORDS = ("off", "exact", "fast", "big")


class ModeError(ValueError):
    """Unknown or undeclared mode word."""


@dataclass(frozen=True)
class ModeSpec:
    name: str
    levers: Tuple[str, ...] = ()
    base: Optional[str] = None          # mode whose lever set this one extends
    note: str = ""


class ModeTable:
    """The modes one kit ships.  ``off`` is mandatory and has no levers."""

    def __init__(self, kit: str, modes: Mapping[str, Sequence[str]], default: Optional[str] = None,
                 bases: Optional[Mapping[str, str]] = None, notes: Optional[Mapping[str, str]] = None):
        if "off" not in modes:
            raise ModeError(f"{kit}: a mode table must contain 'off'")
        if tuple(modes["off"]):
            raise ModeError(f"{kit}: mode 'off' engages nothing")
        for m in modes:
            if m not in MODE_WORDS:
                raise ModeError(f"{kit}: {m!r} is not a mode word ({'|'.join(MODE_WORDS)})")
        if default is not None and default not in modes:
            raise ModeError(f"{kit}: default mode {default!r} is not in the table")
        self.kit = kit
        self.default = default
        self._specs: Dict[str, ModeSpec] = {}
        for m, lv in modes.items():
            self._specs[m] = ModeSpec(m, tuple(lv), (bases or {}).get(m), (notes or {}).get(m, ""))

    def names(self) -> List[str]:
        return [m for m in MODE_WORDS if m in self._specs]

    def __contains__(self, name) -> bool:
        return name in self._specs

    def spec(self, name: str) -> ModeSpec:
        try:
            return self._specs[name]
        except KeyError:
            raise ModeError(f"{self.kit}: unknown mode {name!r}; known: {', '.join(self.names())}") from None

    def levers(self, name: str) -> Tuple[str, ...]:
        """Lever set of a mode, with the base mode's levers first (each once)."""
        spec = self.spec(name)
        out: List[str] = []
        if spec.base:
            out.extend(self.levers(spec.base))
        for lv in spec.levers:
            if lv not in out:
                out.append(lv)
        return tuple(out)


@dataclass(frozen=True)
class Resolution:
    mode: str
    source: str          # "cli" | "env:<NAME>" | "default"
    raw: Optional[str]


def resolve_mode(table: ModeTable, cli_value: Optional[str], env_name: str,
                 environ: Optional[Mapping[str, str]] = None) -> Resolution:
    """CLI > env > default.  A kit without a default and with nothing given is an error."""
    env = os.environ if environ is None else environ
    if cli_value not in (None, ""):
        table.spec(cli_value)
        return Resolution(cli_value, "cli", cli_value)
    ev = (env.get(env_name) or "").strip()
    if ev:
        table.spec(ev)
        return Resolution(ev, f"env:{env_name}", ev)
    if table.default is None:
        raise ModeError(f"{table.kit}: no mode given and the kit has no default; name one of "
                        f"{', '.join(table.names())}")
    return Resolution(table.default, "default", None)


def levers_off(environ: Optional[Mapping[str, str]] = None, name: str = "MODEL_OPT_LEVERS_OFF") -> Tuple[str, ...]:
    """Levers the user switched off by name (comma list in ``MODEL_OPT_LEVERS_OFF``)."""
    env = os.environ if environ is None else environ
    raw = env.get(name) or ""
    return tuple(x.strip() for x in raw.split(",") if x.strip())


def check_declared_env(prefix: str, declared: Iterable[str], environ: Optional[Mapping[str, str]] = None) -> List[str]:
    """Names in the environment that start with ``prefix`` but are not declared by the kit."""
    env = os.environ if environ is None else environ
    declared = set(declared)
    return sorted(k for k in env if k.startswith(prefix) and k not in declared)


class EnvScript:
    """Transcription of a ``configs/<card>.env`` activation script: ordered ``NAME=value`` settings
    (``export`` optional, ``${NAME:-default}`` expanded against the running environment) that can be
    applied to a mapping without a shell."""

    def __init__(self, text: str):
        self.assignments: List[Tuple[str, str]] = []
        for raw in text.splitlines():
            s = raw.strip()
            if not s or s.startswith("#"):
                continue
            if s.startswith("export "):
                s = s[len("export "):].strip()
            if "=" not in s:
                continue
            name, val = s.split("=", 1)
            name = name.strip()
            if not name.replace("_", "a").isalnum():
                continue
            try:
                parts = shlex.split(val, comments=True)
            except ValueError:
                parts = [val]
            self.assignments.append((name, parts[0] if parts else ""))

    @classmethod
    def from_file(cls, path) -> "EnvScript":
        with open(path, "r", encoding="utf-8") as f:
            return cls(f.read())

    @staticmethod
    def _expand(val: str, env: Mapping[str, str]) -> str:
        out, i = "", 0
        while i < len(val):
            if val.startswith("${", i):
                j = val.find("}", i)
                if j < 0:
                    out += val[i:]
                    break
                body = val[i + 2:j]
                if ":-" in body:
                    n, d = body.split(":-", 1)
                    out += env.get(n) or d
                else:
                    out += env.get(body, "")
                i = j + 1
            else:
                out += val[i]
                i += 1
        return out

    def apply(self, environ: Optional[dict] = None, overwrite: bool = False) -> dict:
        env = os.environ if environ is None else environ
        for name, val in self.assignments:
            v = self._expand(val, env)
            if overwrite or name not in env:
                env[name] = v
        return env


def install_env(settings: Mapping[str, str], environ: Optional[dict] = None) -> List[str]:
    """Set variables that are not set yet; returns the names it set."""
    env = os.environ if environ is None else environ
    done = []
    for k, v in settings.items():
        if k not in env:
            env[k] = str(v)
            done.append(k)
    return done
