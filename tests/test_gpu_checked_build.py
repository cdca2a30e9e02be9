"""The checked build of the library (index checks inside the kernels, -DHC_CUDA_CHECKED) on a B200:
every GEMM kernel runs its ladder with the checks compiled in and none fires; the self-test makes one
fire without faulting anything, and the failure arrives as HC_CUDA_ERR_DEVICE_CHECK."""

from __future__ import annotations

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

from hc import cuda
from hc.errors import DeviceError

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parent.parent
CHECKED = REPO / "5_b200" / "lib" / "libhc_cuda_checked.so"

LADDER = textwrap.dedent("""
    import os, sys
    import numpy as np
    from hc import cuda
    from hc.errors import DeviceError

    assert cuda.library_is_checked()
    ctx = cuda.Context(0)
    rng = np.random.default_rng(5)

    def product(m, n, k, dtype=np.float16, pad=0, **kwargs):
        a = (rng.standard_normal((m, k)) * 0.25).astype(dtype)
        b = (rng.standard_normal((k, n)) * 0.25).astype(dtype)
        da, db = ctx.to_device(a), ctx.to_device(b)
        dc = cuda.DeviceBuffer(ctx, (m, n), np.float32, ld=n + pad)
        dc.fill_bytes(0xFF)
        ctx.gemm(da, db, dc, **kwargs)
        ctx.synchronize()  # raises if a check fired
        ref = a.astype(np.float64) @ b.astype(np.float64)
        err = np.linalg.norm(dc.to_numpy() - ref) / np.linalg.norm(ref)
        assert err < 1e-3, (m, n, k, err)
        plan = ctx.plan(m, n, k, "float16", ldc=n + pad)
        for buf in (da, db, dc):
            buf.free()
        return plan

    seen = set()
    for shape in [(100, 300, 200), (128, 256, 64), (515, 770, 96), (1024, 1024, 512), (2048, 2048, 1024),
                  (256, 256, 8192), (512, 512, 4096), (300, 500, 4100), (130, 258, 2050), (4095, 3073, 1031)]:
        for pad in (0, 1):
            plan = product(*shape, pad=pad)
            seen.add((plan.variant, plan.cluster_size > 0, plan.splits > 1))
    os.environ["HC_CUDA_DENSE_WIDE"] = "1"
    assert product(2048, 1024, 4096).tiles_m == 4  # 512-row tiles
    del os.environ["HC_CUDA_DENSE_WIDE"]
    for shape in [(8, 1024, 512), (8, 256, 4096), (33, 512, 2048), (64, 3000, 520), (8, 16384, 256), (1, 1, 1)]:
        plan = product(*shape)
        seen.add((plan.variant, plan.cluster_size > 0, plan.splits > 1))
    assert {("dense", False, False), ("dense", True, True), ("dense", False, True), ("skinny", False, False),
            ("skinny", False, True)} <= seen, seen
    # One check made to fail: reported, nothing faulted, the context still works.
    ctx.selftest_device_check()
    try:
        ctx.synchronize()
    except DeviceError as exc:
        assert exc.status_name == "HC_CUDA_ERR_DEVICE_CHECK" and "index check 99" in str(exc), exc
    else:
        raise AssertionError("the failed check was not reported")
    product(300, 520, 136)
    print("checked ladder ok", sorted(seen))
""")


def test_every_kernel_passes_its_checks_and_a_failing_check_is_reported() -> None:
    assert CHECKED.exists(), "build it with `python 5_b200/build.py --checked`"
    env = dict(os.environ, HC_CUDA_LIB=str(CHECKED),
               PYTHONPATH=os.pathsep.join([str(REPO / "5_b200"), os.environ.get("PYTHONPATH", "")]))
    done = subprocess.run([sys.executable, "-c", LADDER], env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0 and "checked ladder ok" in done.stdout, done.stdout[-2000:] + done.stderr[-4000:]


def test_the_ordinary_build_has_no_checks(gpu_ctx) -> None:
    assert not cuda.library_is_checked()
    with pytest.raises(DeviceError, match="not the checked build"):
        gpu_ctx.selftest_device_check()
