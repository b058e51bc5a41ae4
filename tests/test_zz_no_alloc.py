"""The decode-attention entry point that allocates nothing (csrc/attention_decode_static.h), called through
its exported C symbol: two calls in a row, of different sizes, against the ordinary entry point.

For a caller that cannot hand over scratch memory: the library's own fixed array stands in for it.  The
file is named so that pytest collects it last; it also passes alone in a fresh process."""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(rng, lens, nh, nkv, hd, ps, dtype):
    pages = sum(-(-n // ps) for n in lens) + 3
    pool = (torch.randn(pages, 2, nkv, ps, hd) * 1.5).to(dtype).cuda()
    maxb = max(-(-n // ps) for n in lens)
    bt = np.zeros((len(lens), maxb), dtype=np.int32)
    free = list(rng.permutation(pages))
    for s, n in enumerate(lens):
        for b in range(-(-n // ps)):
            bt[s, b] = free.pop()
    q = (torch.randn(len(lens), nh * hd) * 1.5).to(dtype).cuda()
    seg = torch.arange(len(lens), dtype=torch.int32, device="cuda")
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    return q, pool, torch.from_numpy(bt).cuda(), seg, pos


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_matches_the_ordinary_one(dtype):
    from vitna_anchor_b200 import ops
    lib = ops.lib()
    fn = lib.vk_attention_decode_static
    fn.restype = ctypes.c_int
    rng = np.random.default_rng(12)
    torch.manual_seed(12)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    # two calls in a row with different sizes: the second finds the first one's bytes in the shared array
    for lens, nh, nkv, hd, ps, max_ctx in (([1, 300, 777, 1024, 64], 9, 3, 64, 16, 2048), ([513, 2, 1999], 4, 2, 16, 4, 4096)):
        q, pool, bt, seg, pos = _case(rng, lens, nh, nkv, hd, ps, dtype)
        scale = 1.0 / math.sqrt(hd)
        want = torch.empty_like(q)
        scratch = torch.zeros(ops.attention_decode_scratch_bytes(len(lens), nh, nkv, hd, max_ctx), dtype=torch.uint8, device="cuda")
        ops.attention_decode(q, pool, bt, seg, pos, want, scratch, len(lens), nh, nkv, hd, scale, max_ctx, max_ctx)
        got = torch.full_like(q, 3.0)
        rc = fn(ptr(q), ptr(pool), ptr(bt), ptr(seg), ptr(pos), ctypes.c_void_p(0), ptr(got), len(lens), nh, nkv, hd, ps,
                bt.shape[1], max_ctx, ctypes.c_float(scale), 0, 0 if dtype == torch.float32 else 1, stream)
        assert rc == 0
        torch.cuda.synchronize()
        tol = 1e-5 if dtype == torch.float32 else 2e-2          # the tolerances of the kernel's own test
        assert (got.float() - want.float()).abs().max() <= tol * max(1.0, float(want.float().abs().max()))
    # a launch whose partial results would not fit the library's array is refused before anything runs
    q, pool, bt, seg, pos = _case(rng, [5] * 64, 32, 32, 128, 16, dtype)
    out = torch.empty_like(q)
    rc = fn(ptr(q), ptr(pool), ptr(bt), ptr(seg), ptr(pos), ctypes.c_void_p(0), ptr(out), 64, 32, 32, 128, 16, bt.shape[1],
            32768, ctypes.c_float(0.1), 0, 0 if dtype == torch.float32 else 1, stream)
    assert rc == -3
    err = lib.vk_error_string
    err.restype = ctypes.c_char_p
    assert b"maximum" in err(rc)
