"""mcu_linear_static_scratch: the matmul entry point that allocates nothing.

It serves callers that cannot call cudaMalloc when they need a matmul (all device memory already
reserved by a serving engine or caching allocator, or a thread that cannot take the device-wide
synchronisation an allocation implies).  Its scratch is one fixed array shared by every call, so the
test makes two different calls in a row and checks each against the regular entry point.

Collected last on purpose: a failure here cannot hide failures of the other tests under `-x`.
"""
from __future__ import annotations

import numpy as np
import pytest

from tests.util import KIND_Q4_K, KIND_Q6_K, KIND_Q8_0, TOL_FP32, max_rel_err, random_blocks

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [KIND_Q4_K, KIND_Q6_K, KIND_Q8_0])
def test_static_scratch_matches_mcu_linear_on_two_calls(kind, oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from marmot_b200 import Context
    from marmot_b200.runtime import REGIME_GEMV_PLAIN

    ctx = Context(0)
    lib = ctx.lib
    stream = torch.cuda.current_stream().cuda_stream or 1  # 0x1 = cudaStreamLegacy
    rng = np.random.default_rng(kind)
    # second call: fewer tokens and a shorter, ragged K, so stale bytes of the first call stay in the array
    for T, K, F in [(5, 4096, 200), (2, 1000, 64)]:
        W_host = random_blocks(kind, F, K, rng)
        W = ctx.upload(W_host)
        x_host = rng.normal(0, 1, (T, K)).astype(np.float32)
        bias_host = rng.normal(0, 1, F).astype(np.float32)
        x = torch.from_numpy(x_host).cuda()
        bias = torch.from_numpy(bias_host).cuda()
        out = torch.full((T, F), float("nan"), dtype=torch.float32, device="cuda")
        rc = lib.mcu_linear_static_scratch(stream, kind, x.data_ptr(), K, W.data_ptr(), T, K, F, bias.data_ptr(),
                                           out.data_ptr(), F)
        assert rc == 0, lib.mcu_last_error_message()
        got = out.cpu().numpy()
        ref = ctx.linear(kind, x, W, F, bias=bias).cpu().numpy()
        assert max_rel_err(got, ref) <= TOL_FP32
        # and directly against the CPU oracle of the reference's arithmetic
        assert max_rel_err(got, oracle.linear(kind, x_host, W_host, F, bias=bias_host)) <= TOL_FP32
        # same kernels as the context's plain decode path: identical bits
        ctx.set_regime(REGIME_GEMV_PLAIN)
        plain = ctx.linear(kind, x, W, F, bias=bias).cpu().numpy()
        ctx.set_regime(0)
        assert np.array_equal(got.view(np.uint32), plain.view(np.uint32))
    # beyond the fixed scratch: refused with a clear message, nothing launched
    x = torch.zeros((9, 256), dtype=torch.float32, device="cuda")
    W = ctx.upload(random_blocks(kind, 4, 256, rng))
    out = torch.zeros((9, 4), dtype=torch.float32, device="cuda")
    assert lib.mcu_linear_static_scratch(stream, kind, x.data_ptr(), 256, W.data_ptr(), 9, 256, 4, None,
                                         out.data_ptr(), 4) == -1
    assert b"at most" in lib.mcu_last_error_message()
    assert lib.mcu_linear_static_scratch(stream, kind, x.data_ptr(), 32768, W.data_ptr(), 1, 32768, 4, None,
                                         out.data_ptr(), 4) == -1
    ctx.close()
