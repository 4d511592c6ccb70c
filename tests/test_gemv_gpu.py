"""fp16 GEMV parity: against the fp32-accumulate scalar oracle and against cublasGemmEx called
with the reference's exact arguments (crates/jac-codegen-cuda/src/templates/runtime.cu:18-25).
The reference pins no numerical GEMV vector; tolerance rtol = atol = 1e-2 on fp16 outputs."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import kivi_oracle as ko

pytestmark = pytest.mark.gpu


def _wx(out_dim, in_dim, batch, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((out_dim, in_dim), dtype=np.float32) * 0.02).astype(np.float16)
    x = rng.standard_normal((batch, in_dim), dtype=np.float32).astype(np.float16)
    return w, x


@pytest.mark.parametrize("out_dim,in_dim", [(64, 256), (4096, 128), (1024, 5120), (777, 13824), (7168, 5120)])
@pytest.mark.parametrize("batch", [1, 3, 5, 8, 13, 33, 48, 64])
def test_gemv_matches_oracle(native_lib, out_dim, in_dim, batch):
    from jacq_b200.cache import gemv
    from tests.gpu_utils import f16_tensor
    w, x = _wx(out_dim, in_dim, batch, out_dim + in_dim + batch)
    want16, want32 = ko.gemv(w, x, nthreads=8)
    wd, xd = f16_tensor(w), f16_tensor(x)
    got16 = gemv(wd, xd).cpu().numpy()
    got32 = gemv(wd, xd, out_dtype=torch.float32).cpu().numpy()
    np.testing.assert_allclose(got32, want32, rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(got16.astype(np.float32), want16.astype(np.float32), rtol=1e-2, atol=1e-2)
    # fp32 accumulation in a different order only: far inside the contract's tolerance
    assert np.abs(got32 - want32).max() < 2e-3


def test_gemv_matches_reference_cublas_call(native_lib, ref_lib):
    from jacq_b200.cache import gemv
    from tests.gpu_utils import DEV, f16_tensor, ptr, stream_ptr
    out_dim, in_dim = 5120, 5120
    w, x = _wx(out_dim, in_dim, 1, 3)
    wd, xd = f16_tensor(w), f16_tensor(x[0])
    theirs = torch.zeros(out_dim, dtype=torch.float16, device=DEV)
    rc = ref_lib.ref_gemv_cublas(ptr(wd), ptr(xd), ptr(theirs), ctypes.c_int(in_dim), ctypes.c_int(out_dim), stream_ptr())
    assert rc == 0
    mine = gemv(wd, xd)
    torch.cuda.synchronize()
    np.testing.assert_allclose(mine.cpu().numpy().astype(np.float32), theirs.cpu().numpy().astype(np.float32),
                               rtol=1e-2, atol=1e-2)


def test_gemv_rejects_bad_arguments(native_lib):
    from jacq_b200 import _native
    from jacq_b200.cache import gemv
    from tests.gpu_utils import DEV
    w = torch.zeros((16, 12), dtype=torch.float16, device=DEV)      # in_dim not a multiple of 8
    x = torch.zeros((12,), dtype=torch.float16, device=DEV)
    with pytest.raises(_native.KiviStatusError):
        gemv(w, x)
    with pytest.raises(TypeError):
        gemv(w.float(), x)


def test_skinny_gemm_waits_did_not_fail(native_lib):
    """Every barrier wait of the tcgen05 kernel is bounded and counted when it gives up: after a
    batch that takes that kernel the counter is still zero."""
    from jacq_b200.cache import gemv
    from tests.gpu_utils import f16_tensor
    w, x = _wx(512, 1024, 24, 5)
    gemv(f16_tensor(w), f16_tensor(x))
    failures = ctypes.c_uint32(123)
    assert native_lib.kivi_b200_gemm_wait_failures(ctypes.byref(failures)) == 0
    assert failures.value == 0


_MMA_SYNC_CHECK = """
import numpy as np, torch
from jacq_b200.cache import gemv
from oracle import kivi_oracle as ko
from tests.gpu_utils import f16_tensor
rng = np.random.default_rng(11)
for out_dim, in_dim, batch in [(777, 1024, 13), (1024, 5120, 64), (4096, 128, 8)]:
    w = (rng.standard_normal((out_dim, in_dim), dtype=np.float32) * 0.02).astype(np.float16)
    x = rng.standard_normal((batch, in_dim), dtype=np.float32).astype(np.float16)
    want16, want32 = ko.gemv(w, x, nthreads=8)
    got32 = gemv(f16_tensor(w), f16_tensor(x), out_dtype=torch.float32).cpu().numpy()
    assert np.abs(got32 - want32).max() < 2e-3, (out_dim, in_dim, batch)
print("mma.sync skinny GEMM ok")
"""


def test_mma_sync_skinny_gemm_still_matches(native_lib):
    """The mma.sync kernel that the tcgen05 kernel replaced stays selectable (KIVI_SKINNY_UMMA above 64);
    the switch is read once per process, so the check runs in a child."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    env = dict(os.environ, KIVI_SKINNY_UMMA="99")
    root = Path(__file__).resolve().parent.parent
    done = subprocess.run([sys.executable, "-c", _MMA_SYNC_CHECK], cwd=root, env=env, capture_output=True, text=True,
                          timeout=300)
    assert done.returncode == 0 and "mma.sync skinny GEMM ok" in done.stdout, done.stderr[-2000:]
