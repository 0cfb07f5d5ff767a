"""Split-K decode attention against a plain PyTorch fp32 reference, from one key to tens of thousands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lens", [[1, 63, 700], [9000, 20000], [33000]])
def test_attn_decode_matches_reference(lens):
    from velogb10_b200.ops import kernels as K
    dev = torch.device("cuda")
    torch.manual_seed(len(lens))
    nh, nkv, hd = 6, 2, 256
    n, max_seq = len(lens), max(lens) + 8
    kc = torch.randn(n, nkv, max_seq, hd, device=dev).to(torch.bfloat16)
    vc = torch.randn(n, nkv, max_seq, hd, device=dev).to(torch.bfloat16)
    q = torch.randn(16, nh * hd, device=dev).to(torch.bfloat16)
    lens_t = torch.zeros(16, dtype=torch.int32, device=dev)
    lens_t[:n] = torch.tensor(lens, dtype=torch.int32)
    slots = torch.arange(16, dtype=torch.int32, device=dev) % n
    ns_grid = 32
    part = torch.zeros(K.attn_scratch_floats(16, nh, hd, ns_grid), device=dev)
    out = torch.zeros(16, nh * hd, dtype=torch.float16, device=dev)
    K.attn_decode(q, kc, vc, lens_t, slots, part, out, n, nh, nkv, hd, ns_grid=ns_grid)
    torch.cuda.synchronize()
    G = nh // nkv
    for c, L in enumerate(lens):
        qh = q[c].float().view(nh, hd)
        k = kc[c, :, :L].float().repeat_interleave(G, dim=0)       # [nh, L, hd]
        v = vc[c, :, :L].float().repeat_interleave(G, dim=0)
        p = torch.softmax(torch.einsum("hd,hld->hl", qh, k) / hd ** 0.5, dim=-1)
        ref = torch.einsum("hl,hld->hd", p, v).reshape(-1)
        err = (out[c].float() - ref).abs().max().item()
        assert err < 2e-3 * max(ref.abs().max().item(), 1.0) + 2e-3, (c, L, err)


def _reference(q, k, v, hd):
    """q [nh, hd], k / v [nh, L, hd] fp32 -> [nh * hd]."""
    p = torch.softmax(torch.einsum("hd,hld->hl", q, k) / hd ** 0.5, dim=-1)
    return torch.einsum("hl,hld->hd", p, v).reshape(-1)


@pytest.mark.parametrize("lens,nh,nkv", [([1, 63, 700], 24, 4), ([129, 4096, 300], 16, 2), ([9000, 20000], 24, 4), ([33000], 32, 2)])
def test_tensor_core_decode_attention_matches_reference(lens, nh, nkv):
    """The tcgen05 split-K kernel (one pass over the keys per KV head, whole query group) against fp32 PyTorch, and
    against the CUDA-core kernel's partial statistics."""
    from velogb10_b200.ops import kernels as K, lib
    dev = torch.device("cuda")
    torch.manual_seed(sum(lens))
    hd = 256
    n, max_seq = len(lens), max(lens) + 8
    kc = torch.randn(n, nkv, max_seq, hd, device=dev).to(torch.bfloat16)
    vc = torch.randn(n, nkv, max_seq, hd, device=dev).to(torch.bfloat16)
    q = torch.randn(16, nh * hd, device=dev).to(torch.bfloat16)
    lens_t = torch.zeros(16, dtype=torch.int32, device=dev)
    lens_t[:n] = torch.tensor(lens, dtype=torch.int32)
    slots = torch.arange(16, dtype=torch.int32, device=dev) % n
    part = torch.zeros(K.attn_scratch_floats(16, nh, hd, 32), device=dev)
    part2 = torch.zeros_like(part)
    out = torch.zeros(16, nh * hd, dtype=torch.float16, device=dev)
    out2 = torch.zeros_like(out)
    K.attn_decode_tc(q, kc, vc, lens_t, slots, part, out, n, nh, nkv, hd)
    K.attn_decode(q, kc, vc, lens_t, slots, part2, out2, n, nh, nkv, hd)
    torch.cuda.synchronize()
    lib.check_err_word()
    G = nh // nkv
    pa, pb = part.view(16, nh, 32, hd + 2), part2.view(16, nh, 32, hd + 2)
    for c, L in enumerate(lens):
        ns = max(1, min(32, L // 64))
        # per-split maxima and sums depend on Q K^T only
        assert torch.allclose(pa[c, :, :ns, 0], pb[c, :, :ns, 0], rtol=1e-3, atol=1e-3), ("split maxima", c, L)
        assert torch.allclose(pa[c, :, :ns, 1], pb[c, :, :ns, 1], rtol=2e-2, atol=1e-3), ("split sums", c, L)
        k = kc[c, :, :L].float().repeat_interleave(G, dim=0)
        v = vc[c, :, :L].float().repeat_interleave(G, dim=0)
        ref = _reference(q[c].float().view(nh, hd), k, v, hd)
        err = (out[c].float() - ref).abs().max().item()
        assert err < 4e-3 * max(ref.abs().max().item(), 1.0) + 4e-3, (c, L, err)


def test_tensor_core_decode_attention_over_shared_pages():
    """Block-table addressing: two columns whose tables share their first pages (a common prefix stored once) and then
    diverge give the same result as private copies of the keys."""
    from velogb10_b200.ops import kernels as K, lib
    dev = torch.device("cuda")
    torch.manual_seed(11)
    nh, nkv, hd = 24, 4, 256
    n_pages = 24
    pool_k = torch.randn(n_pages, nkv, 128, hd, device=dev).to(torch.bfloat16)
    pool_v = torch.randn(n_pages, nkv, 128, hd, device=dev).to(torch.bfloat16)
    # column 0: pages 3, 7, 1, 9 (500 keys); column 1: the same first two pages, then 12, 5, 20 (640 keys)
    tables = [[3, 7, 1, 9, 0, 0, 0, 0], [3, 7, 12, 5, 20, 0, 0, 0]]
    lens = [500, 640]
    bt = torch.tensor(tables, dtype=torch.int32, device=dev)
    q = torch.randn(16, nh * hd, device=dev).to(torch.bfloat16)
    lens_t = torch.zeros(16, dtype=torch.int32, device=dev)
    lens_t[:2] = torch.tensor(lens, dtype=torch.int32)
    part = torch.zeros(K.attn_scratch_floats(16, nh, hd, 32), device=dev)
    out = torch.zeros(16, nh * hd, dtype=torch.float16, device=dev)
    K.attn_decode_tc(q, pool_k, pool_v, lens_t, None, part, out, 2, nh, nkv, hd, block_table=bt)
    torch.cuda.synchronize()
    lib.check_err_word()
    G = nh // nkv
    for c, L in enumerate(lens):
        pages = tables[c][:(L + 127) // 128]
        k = torch.cat([pool_k[p] for p in pages], dim=1)[:, :L].float().repeat_interleave(G, dim=0)
        v = torch.cat([pool_v[p] for p in pages], dim=1)[:, :L].float().repeat_interleave(G, dim=0)
        ref = _reference(q[c].float().view(nh, hd), k, v, hd)
        err = (out[c].float() - ref).abs().max().item()
        assert err < 4e-3 * max(ref.abs().max().item(), 1.0) + 4e-3, (c, L, err)
