"""Host side of the guard: deadlines, the error words' meaning, and the test fault injection.

Reference counterpart: ``common/guard.py`` (deadline below the server's watchdog ``:4-7,69``,
error words ``:52-57``, ``fault_injection`` ``:79-88``).  On the device a wait that runs out
stores ``site + 1`` in the deadline word, raises this rank's flag at every peer and the launch
drains; the reference then stops the process by faulting the GPU (``stop_launch`` ``:91-97``),
which this build replaces by an error status the host reads (``mono_guard_read``).

Fault injection is host-side only: ``MONO_FAULT_INJECT=rank:site[:after]`` makes the host of
rank ``rank`` skip the launch that publishes at ``site`` once ``after`` launches of that site
have run, so that every other rank's wait at that site runs out at its deadline.  Nothing on
the device is made to stall, trap or fault.
"""

from __future__ import annotations

import os

ENV = "MONO_FAULT_INJECT"
# the reference refuses a deadline under 5 s and caps it at 60 s (half the watchdog timeout)
MIN_DEADLINE_S, MAX_DEADLINE_S = 5.0, 60.0


def deadline_s(watchdog_timeout_s: float) -> float:
    """Half of the server's watchdog timeout, at most 60 s; under 5 s is refused
    (``common/guard.py:4-7``): a normal delay on one rank must not be a failure."""
    d = min(watchdog_timeout_s / 2.0, MAX_DEADLINE_S)
    if d < MIN_DEADLINE_S:
        raise ValueError(f"a watchdog timeout of {watchdog_timeout_s} s leaves a {d} s wait deadline; needs at least "
                         f"{2 * MIN_DEADLINE_S} s")
    return d


def fault_injection(rank: int):
    """(site, after) when ``MONO_FAULT_INJECT`` names this rank, else None."""
    spec = os.environ.get(ENV, "")
    if not spec:
        return None
    r, site, after = (spec.split(":") + ["0", "0"])[:3]
    return (int(site or 0), int(after or 0)) if int(r) == rank else None


class FaultInjector:
    """Counts this rank's launches per site and says when the host must skip one."""

    def __init__(self, rank: int):
        self.spec = fault_injection(rank)
        self.count = 0

    def skip(self, site: int) -> bool:
        if self.spec is None or site != self.spec[0]:
            return False
        self.count += 1
        return self.count > self.spec[1]
