"""Stand-in for the `greenlet` package (test infrastructure only).

The reference simulator runs each workitem of an `@group.workitems` region as a greenlet so
that `group.barrier()` can suspend it (hc/simulator.py:560-654). The matmul example never
calls a barrier, so a coroutine that simply runs to completion on its first `switch` is
enough to execute it unmodified. A workitem that does try to yield to the scheduler (a
barrier) is reported as unsupported rather than mis-simulated. Nothing in the product
imports this module.
"""

from __future__ import annotations


class _Root:
    dead = False

    def switch(self, *args, **kwargs):
        raise RuntimeError(
            "the greenlet stand-in cannot suspend a workitem (group.barrier() is not supported)"
        )


_ROOT = _Root()


def getcurrent():
    return _ROOT


class greenlet:  # noqa: N801 - mirrors the real package's class name
    def __init__(self, run=None, parent=None):
        self.run = run
        self.parent = parent
        self.dead = False

    def switch(self, *args, **kwargs):
        if self.dead:
            raise RuntimeError("cannot switch to a finished greenlet")
        try:
            return self.run(*args, **kwargs)
        finally:
            self.dead = True
