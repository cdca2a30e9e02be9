"""Exception classes of the launch path.

The reference raises `LaunchError` (a `SimulatorError`, hc/_sim_types.py:62-67) for every
problem found while preparing a launch: a non-array buffer, a rank or dtype that does not
match the `Buffer` annotation, contradictory symbol bindings, bad launch geometry
(hc/simulator.py:189-229, 752-768, 858-900). The compiled NVIDIA path raises the same class
names with the same message texts so that callers and tests written against the simulator
keep working. `DeviceError` is new: a failure reported by the CUDA library.
"""

from __future__ import annotations


class SimulatorError(RuntimeError):
    pass


class LaunchError(SimulatorError):
    pass


class DeviceError(RuntimeError):
    """A call into the CUDA library failed. `status` is the HcCudaStatus code."""

    def __init__(self, status: int, status_name: str, detail: str) -> None:
        super().__init__(f"{status_name}: {detail}" if detail else status_name)
        self.status = status
        self.status_name = status_name
        self.detail = detail
