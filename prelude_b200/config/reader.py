"""Reading the keys of a layer-by-layer config.json: every problem is collected and named, none stops the parse."""
from __future__ import annotations

import math


def _is_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v)


class _Reader:
    """Reads keys of one JSON object and collects what is wrong with them."""

    def __init__(self, raw, where: str, problems: list):
        self.raw = raw if isinstance(raw, dict) else {}
        self.where, self.problems = where, problems
        if not isinstance(raw, dict):
            problems.append(f"{where} must be an object")

    def _get(self, key):
        if key not in self.raw or self.raw[key] is None:
            self.problems.append(f"{self.where}: missing field `{key}`")
            return None
        return self.raw[key]

    def positive_int(self, key) -> int:
        v = self._get(key)
        if v is not None and (not _is_int(v) or v <= 0):
            self.problems.append(f"{self.where}: `{key}` must be a positive integer, got {v!r}")
            v = None
        return v if v is not None else 1

    def number(self, key, positive: bool = False) -> float:
        v = self._get(key)
        if v is not None and (not _is_num(v) or (positive and v <= 0)):
            self.problems.append(f"{self.where}: `{key}` must be a {'positive ' if positive else ''}number, got {v!r}")
            v = None
        return float(v) if v is not None else 1.0

    def obj(self, key) -> "_Reader":
        v = self._get(key)
        return _Reader({} if v is None else v, f"{self.where}.{key}", self.problems)
