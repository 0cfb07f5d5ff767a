"""The allocation-free attention entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory when they need attention (they run under an
allocator lock, or gave all of their HBM away at start-up), so ``vg_attn_decode_static`` keeps its split-K
partials in an array inside the library image. The test drives it through ctypes exactly as such a caller
would, twice in a row with different inputs, and requires the same output as the regular entry point that
takes a caller-provided partial buffer. It also checks that an oversized request is refused.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, n, lens, nh=8, nkv=2, hd=128, max_seq=1024, slots=2):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(n, nh, hd, generator=g, device="cuda").to(torch.bfloat16)
    kc = torch.randn(slots, nkv, max_seq, hd, generator=g, device="cuda").to(torch.bfloat16)
    vc = torch.randn(slots, nkv, max_seq, hd, generator=g, device="cuda").to(torch.bfloat16)
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    slot_t = torch.tensor([i % slots for i in range(n)], dtype=torch.int32, device="cuda")
    return q, kc, vc, lens_t, slot_t


def test_static_scratch_entry_matches_regular_entry_twice():
    from velogb10_b200.ops import build
    build.build()
    L = ctypes.CDLL(build.LIB_PATH)
    L.vg_attn_scratch_floats.restype = ctypes.c_longlong
    vp, ci = ctypes.c_void_p, ctypes.c_int
    st = vp(torch.cuda.current_stream().cuda_stream)
    max_seq = 1024
    # (the last case is the model shape, head_dim 256, with fewer splits than the columns' lengths ask for)
    for seed, n, lens, nh, nkv, hd, ns in ((1, 3, [5, 700, 1024], 8, 2, 128, 32), (2, 5, [300, 1, 513, 256, 999], 8, 2, 128, 32),
                                           (3, 2, [1024, 130], 6, 2, 256, 4)):
        q, kc, vc, lens_t, slot_t = _case(seed, n, lens, nh, nkv, hd, max_seq)
        part = torch.empty(int(L.vg_attn_scratch_floats(ci(n), ci(nh), ci(hd), ci(ns))), dtype=torch.float32, device="cuda")
        ref = torch.zeros(n, nh * hd, dtype=torch.float16, device="cuda")
        got = torch.zeros_like(ref)
        rc = L.vg_attn_decode(vp(q.data_ptr()), vp(kc.data_ptr()), vp(vc.data_ptr()), vp(lens_t.data_ptr()),
                              vp(slot_t.data_ptr()), vp(0), vp(0), ci(0), vp(part.data_ptr()), ci(n), ci(nh), ci(nkv),
                              ci(hd), ci(max_seq), ci(ns), ci(0), vp(0), ci(0), vp(ref.data_ptr()), st)
        assert rc == 0
        rc = L.vg_attn_decode_static(vp(q.data_ptr()), vp(kc.data_ptr()), vp(vc.data_ptr()), vp(lens_t.data_ptr()),
                                     vp(slot_t.data_ptr()), vp(0), vp(0), ci(0), ci(n), ci(nh), ci(nkv), ci(hd),
                                     ci(max_seq), ci(ns), ci(0), vp(0), ci(0), vp(got.data_ptr()), st)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.allclose(got.float(), ref.float(), rtol=1e-3, atol=1e-3)
        # and against a plain fp32 reference of the op
        for c in range(n):
            s = int(slot_t[c])
            K = kc[s, :, :lens[c]].float().repeat_interleave(nh // nkv, 0)
            V = vc[s, :, :lens[c]].float().repeat_interleave(nh // nkv, 0)
            p = torch.softmax(torch.einsum("hd,htd->ht", q[c].float(), K) / hd ** 0.5, -1)
            want = torch.einsum("ht,htd->hd", p, V).reshape(-1)
            assert torch.allclose(got[c].float(), want, rtol=2e-2, atol=2e-2)
    # a request larger than the built-in buffer is refused and launches nothing
    rc = L.vg_attn_decode_static(vp(0), vp(0), vp(0), vp(0), vp(0), vp(0), vp(0), ci(0), ci(4096), ci(32), ci(8), ci(256),
                                 ci(max_seq), ci(32), ci(0), vp(0), ci(0), vp(0), st)
    assert rc == -20
    torch.cuda.synchronize()
