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
