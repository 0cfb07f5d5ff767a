"""Tensor-core and CUDA-core GEMM kernels against a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(fmt, m, k, seed=0):
    from velogb10_b200.models.weights import QLinear
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = (torch.randn(m, k, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
    return QLinear.from_dense(w, fmt)


def _ref(q, x16):
    return x16.float() @ q.dequant(torch.float32).t()


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8", "bf16"])
@pytest.mark.parametrize("m,k,n", [(128, 128, 1), (256, 256, 16), (384, 1024, 5), (1552, 256, 3),
                                   (5120, 5120, 16), (640, 2048, 40), (512, 640, 100), (1024, 512, 300),
                                   (19072, 640, 300), (38016, 384, 700)])   # the last two take the 256-token tile
def test_gemm_tc_matches_reference(fmt, m, k, n):
    from velogb10_b200.ops import gemm as G, lib
    q = _mk(fmt, m, k)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(max(n, 16), k, generator=g, device="cuda").to(torch.float16)
    out = G.linear(q, x, n, out_f32=True)
    torch.cuda.synchronize()
    lib.check_err_word()
    ref = _ref(q, x[:n])
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 2e-3 * scale + 1e-4, (err, scale)
    out_bf = G.linear(q, x, n)
    assert (out_bf.float() - ref).abs().max().item() <= 1e-2 * scale + 1e-3


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8", "bf16"])
def test_gemm_simt_matches_reference(fmt):
    from velogb10_b200.ops import gemm as G
    q = _mk(fmt, 272, 784 if fmt != "nvfp4" else 784 - 16)
    x = torch.randn(16, q.k, device="cuda").to(torch.float16)
    out = G.linear_simt(q, x, 7, out_f32=True)
    ref = _ref(q, x[:7])
    assert (out - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-4


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8"])
@pytest.mark.parametrize("m,k", [(5120, 17408), (1024, 5120), (2176, 640)])
def test_gemm_tc_batch_invariant(fmt, m, k):
    """Column 0 of a width-N call has the same bits for every N in 1..16, and the call is deterministic."""
    from velogb10_b200.ops import gemm as G
    q = _mk(fmt, m, k)
    x = torch.randn(16, k, device="cuda").to(torch.float16)
    base = G.linear(q, x, 1, out_f32=True).clone()
    for n in range(1, 17):
        out = G.linear(q, x, n, out_f32=True)
        assert torch.equal(out[0], base[0]), n
    again = G.linear(q, x, 16, out_f32=True).clone()
    assert torch.equal(again, G.linear(q, x, 16, out_f32=True))
    # every column equals the same data placed in column 0
    full = G.linear(q, x, 16, out_f32=True).clone()
    for c in (3, 15):
        xs = x.clone()
        xs[0] = x[c]
        assert torch.equal(G.linear(q, xs, 1, out_f32=True)[0], full[c])


def test_splitk_choice_is_width_independent():
    from velogb10_b200.ops import gemm as G
    assert 1 <= G.choose_splitk(5120, 17408, 0) <= 8
    assert G.choose_splitk(5120, 17408, 0) == G.choose_splitk(5120, 17408, 0)


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8", "bf16"])
@pytest.mark.parametrize("m,k", [(5120, 5120), (640, 1664)])
def test_gemm_tc_every_splitk(fmt, m, k):
    """Every cluster split-K factor gives the reference result (odd and even slab counts per CTA)."""
    from velogb10_b200.ops import gemm as G, lib
    q = _mk(fmt, m, k)
    G.prepare(q)
    x = torch.randn(16, k, device="cuda").to(torch.float16)
    ref = _ref(q, x)
    for s in range(1, 9):
        q.kernel.splitk = s
        out = G.linear(q, x, 16, out_f32=True)
        torch.cuda.synchronize()
        lib.check_err_word()
        err = (out - ref).abs().max().item()
        assert err <= 2e-3 * ref.abs().max().item() + 1e-4, (s, err)
