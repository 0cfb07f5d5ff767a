"""Block-scaled FP4 tensor-core GEMM (weights consumed packed, activations as a four-term NVFP4 series)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(m, k, seed=0):
    from velogb10_b200.models.weights import QLinear
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(m, k, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    return QLinear.from_dense(w, "nvfp4")


@pytest.mark.parametrize("m,k,n", [(128, 256, 1), (256, 512, 16), (384, 1024, 5), (1552, 256, 3), (5120, 5120, 16),
                                   (640, 2176, 7), (5120, 17408, 2),
                                   (76032, 512, 3), (80000, 768, 16), (75904, 1280, 1)])   # deep tile loops: persistent kernel
def test_fp4_gemm_matches_reference(m, k, n):
    from velogb10_b200.ops import gemm as G, lib
    q = _mk(m, k)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(16, k, generator=g, device="cuda").to(torch.float16)
    x[0, ::7] *= 30.0                                   # wide dynamic range inside a column
    out = G.linear_fp4(q, x, n, out_f32=True)
    torch.cuda.synchronize()
    lib.check_err_word()
    ref = x[:n].float() @ q.dequant(torch.float32).t()
    rel = ((out - ref).norm() / ref.norm()).item()
    assert rel < 3e-3, rel


def test_fp4_gemm_batch_invariant_and_splitk():
    from velogb10_b200.ops import gemm as G
    q = _mk(5120, 6144)
    x = torch.randn(16, 6144, device="cuda").to(torch.float16)
    base = G.linear_fp4(q, x, 1, out_f32=True).clone()
    full = G.linear_fp4(q, x, 16, out_f32=True).clone()
    for n in range(1, 17):
        assert torch.equal(G.linear_fp4(q, x, n, out_f32=True)[0], base[0]), n
    xs = x.clone()
    xs[0] = x[9]
    assert torch.equal(G.linear_fp4(q, xs, 1, out_f32=True)[0], full[9])
    ref = x.float() @ q.dequant(torch.float32).t()
    for s in range(1, 9):
        q.kernel4.splitk = s
        out = G.linear_fp4(q, x, 16, out_f32=True)
        assert ((out - ref).norm() / ref.norm()).item() < 3e-3, s


@pytest.mark.parametrize("h,n", [(5120, 1), (2048, 16), (256, 5), (17408, 3)])
def test_fused_rmsnorm_quantiser(h, n):
    """RMSNorm that emits the FP4 series directly feeds the GEMM like norm -> f16 -> quantise does."""
    from velogb10_b200.ops import gemm as G, kernels as K, lib
    q = _mk(384, h)
    res = (torch.randn(16, h, device="cuda") * 2).to(torch.bfloat16)
    delta = torch.randn(16, h, device="cuda").to(torch.bfloat16)
    w = torch.randn(h, device="cuda") * 0.1
    r1, r2 = res.clone(), res.clone()
    x16a = torch.zeros(16, h, dtype=torch.float16, device="cuda")
    x16b = torch.zeros_like(x16a)
    K.add_rmsnorm(r1, delta, w, 1e-6, n, out16=x16a)
    want = G.linear_fp4(q, x16a, n, out_f32=True).clone()
    act = G.add_rmsnorm_fp4(r2, delta, w, 1e-6, n, out16=x16b)
    got = G.linear_fp4(q, x16b, n, out_f32=True, act=act)
    torch.cuda.synchronize()
    lib.check_err_word()
    assert torch.equal(r1[:n], r2[:n])
    assert (x16a[:n].float() - x16b[:n].float()).abs().max() <= 2e-3 * x16a[:n].float().abs().max()
    xs = (res[:n].float() + delta[:n].float()).to(torch.bfloat16).float()
    ref = (xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + 1e-6) * (1 + w)) @ q.dequant(torch.float32).t()
    assert ((got - ref).norm() / ref.norm()).item() < 4e-3
    assert ((got - want).norm() / ref.norm()).item() < 2e-3


@pytest.mark.parametrize("inter,n", [(17408, 1), (1024, 16), (768, 4)])
def test_fused_swiglu_quantiser(inter, n):
    from velogb10_b200.ops import gemm as G, kernels as K, lib
    q = _mk(256, inter)
    gu = torch.randn(16, 2 * inter, device="cuda").to(torch.bfloat16)
    a16 = torch.zeros(16, inter, dtype=torch.float16, device="cuda")
    K.swiglu(gu, a16, n, inter)
    want = G.linear_fp4(q, a16, n, out_f32=True).clone()
    act = G.swiglu_fp4(gu, n, inter)
    got = G.linear_fp4(q, a16, n, out_f32=True, act=act)
    torch.cuda.synchronize()
    lib.check_err_word()
    assert torch.equal(got, want)


def test_grouped_fp4_matches_reference():
    """MoE decode form: each work item multiplies one expert with one activation row and writes one output row."""
    from velogb10_b200.models.weights import QLinear
    from velogb10_b200.ops import gemm as G, lib
    E, M, K, n_tok, topk = 6, 256, 512, 3, 4
    g = torch.Generator(device="cuda").manual_seed(3)
    w = (torch.randn(E * M, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    q = QLinear.from_dense(w, "nvfp4")
    wd = q.dequant(torch.float32).view(E, M, K)
    x = torch.randn(16, K, generator=g, device="cuda").to(torch.float16)
    act = G.quantize_act_fp4(x, n_tok, K)
    P = n_tok * topk
    ids = torch.tensor([0, 5, 2, 3, 1, 4, 0, 2, 5, 5, 3, 1], dtype=torch.int32, device="cuda")
    g_exp = ids.clone()
    g_exp[7] = -1                                            # a non-resident expert: row must stay untouched
    g_off = torch.arange(P, dtype=torch.int32, device="cuda")
    out = torch.full((P, M), 7.0, dtype=torch.bfloat16, device="cuda")
    G.linear_fp4_grouped(q, act, out, g_exp, g_off, P, topk, M)
    # second stage shape: one quantised row per pair (more than 16 rows -> several B tiles)
    P2 = 40
    y = torch.randn(P2, K, generator=g, device="cuda").to(torch.float16)
    bufs = G.fp4_buffers("cuda", K, rows=P2, tag="test")
    rc = lib.lib().vg_act_quant_fp4(lib.ptr(y), lib.c_int(y.stride(0)), lib.c_int(P2), lib.c_int(K), lib.ptr(bufs[0]),
                                    lib.c_int(bufs[0].stride(0)), lib.ptr(bufs[1]), lib.ptr(bufs[2]), lib.stream())
    assert rc == 0
    ids2 = torch.randint(0, E, (P2,), generator=torch.Generator().manual_seed(1)).to(torch.int32).cuda()
    off2 = torch.arange(P2, dtype=torch.int32, device="cuda")
    out2 = torch.zeros((P2, M), dtype=torch.float32, device="cuda")
    G.linear_fp4_grouped(q, bufs, out2, ids2, off2, P2, 1, M)
    torch.cuda.synchronize()
    lib.check_err_word()
    for p_ in range(P):
        if p_ == 7:
            assert torch.all(out[p_].float() == 7.0)
            continue
        ref = wd[int(ids[p_])] @ x[p_ // topk].float()
        rel = ((out[p_].float() - ref).norm() / ref.norm()).item()
        assert rel < 8e-3, (p_, rel)
    ref2 = torch.einsum("pmk,pk->pm", wd[ids2.long()], y.float())
    assert ((out2 - ref2).norm() / ref2.norm()).item() < 3e-3
