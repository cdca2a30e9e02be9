"""The compile-time probe model (`hc._tile_probe`): the few workgroup calls it covers behave as the
reference simulator's do (masked loads hc/simulator.py:1338-1357, clipped stores :1441-1458, per-lane
results stacked along (wave, 1) :292-300)."""

import numpy as np
import pytest

from hc._tile_probe import ProbeError, ProbeGroup, ProbeValue


def test_load_masks_what_lies_outside_the_buffer() -> None:
    group = ProbeGroup((0, 0), 4, (4, 1))
    buffer = np.arange(12, dtype=np.float32).reshape(3, 4)
    tile = group.load(buffer[1:5, 2:6], shape=(4, 4))  # NumPy clips the window to 2 x 2
    assert tile.shape == (4, 4) and tile.dtype == np.float32
    assert tile[0, 1] == 7.0 and tile[1, 0] == 10.0
    with pytest.raises(ProbeError, match="inactive"):
        tile[2, 0]
    filled = tile.with_inactive(value=np.float32(-1))
    assert filled[3, 3] == -1.0 and filled[0, 0] == 6.0
    row = tile[0, :].vec().with_inactive(value=np.float32(0))
    assert [row[i] for i in range(4)] == [6.0, 7.0, 0.0, 0.0]
    with pytest.raises(TypeError):
        np.asarray(tile)
    with pytest.raises(ProbeError, match="shape"):
        group.load(buffer[0:2, 0:2])


def test_store_writes_the_active_overlap_only() -> None:
    group = ProbeGroup((0, 0), 4, (4, 1))
    target = np.zeros((3, 3), np.float32)
    value = group.load(np.full((2, 5), 9, np.float32), shape=(4, 5))  # rows 2.. are inactive
    group.store(target[1:, 1:], value)
    assert target.tolist() == [[0, 0, 0], [0, 9, 9], [0, 9, 9]]
    group.store(target[3:, :], value)  # empty overlap at the edge: nothing happens
    with pytest.raises(ProbeError, match="ranks"):
        group.store(target[0], value)


def test_workitems_stack_lane_results_and_arithmetic_keeps_masks() -> None:
    group = ProbeGroup((2, 1), 4, (12, 2))

    @group.workitems
    def per_lane(wi):
        lane = wi.local_id()[0]
        assert wi.global_id() == (8 + lane, 1)
        return group.vfull(shape=(3,), dtype=np.float32, fill_value=lane)

    stacked = per_lane()
    assert stacked.shape == (3, 4, 1)
    assert [stacked[0, lane, 0] for lane in range(4)] == [0.0, 1.0, 2.0, 3.0]
    doubled = stacked[:, 2, 0] * 2 + 1
    assert isinstance(doubled, ProbeValue) and doubled[1] == 5.0
    half = group.load(np.ones((2,), np.float32), shape=(3,))
    total = stacked[:, 1, 0] + half
    assert total[0] == 2.0
    with pytest.raises(ProbeError, match="inactive"):
        total[2]

    @group.workitems
    def nothing(wi):
        return None

    assert nothing() is None
    with pytest.raises(ProbeError, match="barrier"):
        group.barrier()
