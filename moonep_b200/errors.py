"""Errors raised when a kernel reports a problem through the status block."""

from __future__ import annotations


class MoonEPError(RuntimeError):
    pass


class MoonEPTimeoutError(MoonEPError):
    """A bounded device-side wait ran out: a peer never produced the flag a kernel was waiting for."""

    def __init__(self, msg, *, kernel=None, family=None, peer=None, expected=None, seen=None):
        super().__init__(msg)
        self.kernel, self.family, self.peer, self.expected, self.seen = kernel, family, peer, expected, seen


class MoonEPIndexError(MoonEPError):
    """A kernel met an index outside its buffer (corrupt plan or routing input) and skipped the access."""
