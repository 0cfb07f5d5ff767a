"""Tensor-core prefill attention against a plain fp32 reference (causal, GQA, chunk after cached context)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pos0,n,gated", [(0, 128, False), (0, 300, True), (200, 333, True), (512, 77, False)])
def test_prefill_attention_matches_reference(pos0, n, gated):
    from velogb10_b200.ops import kernels as K, lib
    torch.manual_seed(pos0 + n)
    dev = "cuda"
    nh, nkv, hd, max_seq, slots, slot = 6, 2, 256, 1024, 3, 1
    cap = 512
    q = torch.randn(cap, nh * hd, device=dev).to(torch.bfloat16)
    kc = torch.zeros(slots, nkv, max_seq, hd, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    L = pos0 + n
    kc[slot, :, :L] = torch.randn(nkv, L, hd, device=dev).to(torch.bfloat16)
    vc[slot, :, :L] = torch.randn(nkv, L, hd, device=dev).to(torch.bfloat16)
    qkv = torch.randn(cap, nh * hd * 2 + 64, device=dev).to(torch.bfloat16)       # gate of head h at h*2hd + hd
    vT = torch.zeros(nkv, hd, max_seq, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(cap, nh * hd, dtype=torch.float16, device=dev)
    K.attn_prefill_tc(q, kc, vc, vT, slot, pos0, n, nh, nkv, hd, out, gate=qkv if gated else None)
    torch.cuda.synchronize()
    lib.check_err_word()

    qf = q[:n].float().view(n, nh, hd)
    G = nh // nkv
    kf = kc[slot, :, :L].float().repeat_interleave(G, 0)            # [nh, L, hd]
    vf = vc[slot, :, :L].float().repeat_interleave(G, 0)
    s = torch.einsum("nhd,hld->hnl", qf, kf) * hd ** -0.5
    qpos = pos0 + torch.arange(n, device=dev)
    mask = torch.arange(L, device=dev)[None, :] > qpos[:, None]
    s = s.masked_fill(mask[None], float("-inf"))
    ref = torch.einsum("hnl,hld->nhd", torch.softmax(s, -1), vf)
    if gated:
        gate = qkv[:n].float()[:, :nh * hd * 2].view(n, nh, 2 * hd)[:, :, hd:]
        ref = ref * torch.sigmoid(gate)
    got = out[:n].float().view(n, nh, hd)
    rel = ((got - ref).norm() / ref.norm()).item()
    assert rel < 8e-3, rel
    assert (got - ref).abs().max().item() < 0.05
