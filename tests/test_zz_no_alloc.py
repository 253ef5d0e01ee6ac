"""ff_shared_ffn_noalloc: the shared INT4 FFN for callers that cannot allocate device memory
(a decode loop where cudaMalloc would stall the GPU, or a process whose HBM another runtime has
already reserved).
Its activations scratch is a fixed array inside the library; this test drives it through the
C ABI and checks it against the context-based ff_shared_ffn on the same weights, twice in a row
(the second call reuses the array with the first call's contents still in it), against the CPU
oracle, and at the corner of its documented limits (16 rows, intermediate width 4096)."""
import ctypes

import numpy as np
import pytest

from ane_fieldfare_b200 import binding, gturbo, workload
from conftest import assert_layer_close, oracle_layer

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _device_projections(hp, L, device):
    keep, projs = [], []
    for role in gturbo.ROLES:
        w, s, b = gturbo.sub_tensor(L.sharedBlob, L.sharedLayout, role)
        rows, cols = L.sharedLayout.matrix_shape(role)
        wd = torch.from_numpy(np.ascontiguousarray(w)).to(device)
        sd = hp.bf16_tensor(np.ascontiguousarray(s), device)
        bd = hp.bf16_tensor(np.ascontiguousarray(b), device)
        keep += [wd, sd, bd]
        projs.append(binding.FFProjection(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), rows, cols))
    return keep, projs


def _noalloc(projs, x, rows, d, got, stream):
    binding.call("ff_shared_ffn_noalloc", ctypes.byref(projs[0]), ctypes.byref(projs[1]),
                 ctypes.byref(projs[2]), x.data_ptr(), d, rows, got.data_ptr(), d, stream)


def test_noalloc_shared_ffn_matches_context_path_twice(oracle):
    from ane_fieldfare_b200 import hotpath as hp
    L = workload.make_layer(0x40A110C, 0, experts=8, d=256, f=64, sharedF=320, topK=4)
    ctx = hp.HotpathContext(layers=1, experts=8, d=256, f=64, sharedF=320, topK=4, maxTokens=16)
    try:
        workload.load_layer(ctx, 0, L)
        device = ctx.device
        keep, projs = _device_projections(hp, L, device)
        stream = torch.cuda.current_stream().cuda_stream or None
        for call_index, rows in enumerate((16, 5, 1)):
            bits = workload.make_tokens(7 + call_index, "noalloc", rows, 256)
            x = hp.bf16_tensor(bits, device)
            want = torch.zeros((rows, 256), dtype=torch.bfloat16, device=device)
            hp.SharedExpertInt4(ctx).encode(None, 0, x, want, rows=rows)
            got = torch.full((rows, 256), 7.0, dtype=torch.bfloat16, device=device)
            _noalloc(projs, x, rows, 256, got, stream)
            torch.cuda.synchronize()
            assert torch.isfinite(got.float()).all()
            diff = (got.float() - want.float()).abs().max().item()
            peak = max(1.0, want.float().abs().max().item())
            assert diff <= 2e-2 * peak, (call_index, diff)
            # two rows and more take the same GEMV kernels in both entry points: the same bits; one
            # row goes through the fused decode kernel in ff_shared_ffn (another summation order)
            if rows > 1:
                assert torch.equal(got, want), f"call {call_index}: not bitwise the context path"
            assert_layer_close(hp.bf16_numpy(got), oracle.shared_ffn(oracle_layer(oracle, L), bits), oracle,
                               f"noalloc shared FFN rows={rows}")
        # sizes beyond the static scratch are refused with a message
        with pytest.raises(binding.FieldfareError, match="at most 16 rows"):
            binding.call("ff_shared_ffn_noalloc", ctypes.byref(projs[0]), ctypes.byref(projs[1]),
                         ctypes.byref(projs[2]), x.data_ptr(), 256, 17, got.data_ptr(), 256, stream)
        wide = binding.FFProjection(projs[0].weights, projs[0].scales, projs[0].biases, 8192, 256)
        with pytest.raises(binding.FieldfareError, match="exceeds the static scratch"):
            binding.call("ff_shared_ffn_noalloc", ctypes.byref(wide), ctypes.byref(projs[1]),
                         ctypes.byref(projs[2]), x.data_ptr(), 256, 4, got.data_ptr(), 256, stream)
    finally:
        ctx.close()


def test_noalloc_at_the_corner_of_its_limits(oracle):
    """16 rows with the largest intermediate width the static scratch holds (4096): the 16 staged
    rows of the down projection do not fit in shared memory together, so it runs as two passes of
    eight; the bits are those of the context path, which splits the same way."""
    from ane_fieldfare_b200 import hotpath as hp
    L = workload.make_layer(0x40A110D, 0, experts=8, d=256, f=64, sharedF=4096, topK=4)
    ctx = hp.HotpathContext(layers=1, experts=8, d=256, f=64, sharedF=4096, topK=4, maxTokens=16)
    try:
        workload.load_layer(ctx, 0, L)
        keep, projs = _device_projections(hp, L, ctx.device)
        stream = torch.cuda.current_stream().cuda_stream or None
        bits = workload.make_tokens(11, "noalloc.corner", 16, 256)
        x = hp.bf16_tensor(bits, ctx.device)
        for attempt in range(2):
            got = torch.full((16, 256), 7.0, dtype=torch.bfloat16, device=ctx.device)
            _noalloc(projs, x, 16, 256, got, stream)
            torch.cuda.synchronize()
            assert_layer_close(hp.bf16_numpy(got), oracle.shared_ffn(oracle_layer(oracle, L), bits), oracle,
                               f"noalloc corner 16 x 4096, call {attempt}")
        want = torch.zeros((16, 256), dtype=torch.bfloat16, device=ctx.device)
        hp.SharedExpertInt4(ctx).encode(None, 0, x, want, rows=16)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    finally:
        ctx.close()
