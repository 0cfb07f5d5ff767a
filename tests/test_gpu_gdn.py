"""GatedDeltaNet recurrence kernels: the batched prefill kernel reproduces the per-token step kernel bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T", [17, 64, 333])
def test_prefill_kernel_matches_step_kernel_bitwise(T):
    from velogb10_b200.ops import kernels as K, lib
    torch.manual_seed(T)
    dev = "cuda"
    nk, nv, kd, vd = 2, 6, 128, 128
    key_dim, value_dim = nk * kd, nv * vd
    conv_dim = 2 * key_dim + value_dim
    ldp = (conv_dim + value_dim + 2 * nv + 7) // 8 * 8      # rows start on 16-byte boundaries (async copies)
    qkv = torch.randn(T, conv_dim, device=dev)
    proj = torch.randn(T, ldp, device=dev).to(torch.bfloat16)
    A_log = torch.randn(nv, device=dev) * 0.5
    dt_bias = torch.randn(nv, device=dev) * 0.5
    norm_w = torch.rand(vd, device=dev) + 0.5
    S0 = torch.randn(3, nv, kd, vd, device=dev) * 0.1
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    in_slot = i32([1] * T)
    parent = i32([-1] + list(range(T - 1)))
    out_slot = i32([-1] * (T - 1) + [2])
    out_slot[T // 2] = 0                                    # a checkpoint in the middle of the chain
    chain_start, chain_len = i32([0]), i32([T])

    Sa, Sb = S0.clone(), S0.clone()
    oa = torch.zeros(T, nv * vd, dtype=torch.float16, device=dev)
    ob = torch.zeros_like(oa)
    K.gdn_step(qkv, proj, conv_dim, conv_dim + value_dim, conv_dim + value_dim + nv, Sa, A_log, dt_bias, norm_w,
               chain_start, chain_len, 1, in_slot, parent, out_slot, oa, nk, nv, kd, vd, 1e-6)
    K.gdn_prefill(qkv, proj, conv_dim, conv_dim + value_dim, conv_dim + value_dim + nv, Sb, A_log, dt_bias, norm_w,
                  0, T, in_slot, out_slot, ob, nk, nv, kd, vd, 1e-6)
    torch.cuda.synchronize()
    lib.check_err_word()
    assert torch.equal(oa, ob)
    assert torch.equal(Sa, Sb)
    # column-split forms (2 and 4 CTAs per head + separate output norm): same bits
    scratch = torch.zeros(T * nv * vd, device=dev)
    for split in (2, 4):
        Sc = S0.clone()
        oc = torch.zeros_like(oa)
        K.gdn_prefill(qkv, proj, conv_dim, conv_dim + value_dim, conv_dim + value_dim + nv, Sc, A_log, dt_bias, norm_w,
                      0, T, in_slot, out_slot, oc, nk, nv, kd, vd, 1e-6, o_scratch=scratch, split=split)
        torch.cuda.synchronize()
        assert torch.equal(oa, oc) and torch.equal(Sa, Sc), split


@pytest.mark.parametrize("n", [1, 3, 50, 256])
def test_conv_chain_matches_two_phase_conv_bitwise(n):
    """The prefill conv (eight channels per thread, window in registers) against the generic per-element kernel:
    same outputs and same carried state, bit for bit; and against a plain fp32 reference."""
    from velogb10_b200.ops import kernels as K
    dev = torch.device("cuda")
    torch.manual_seed(3)
    conv_dim, ck, ldx, slots = 1032, 4, 1048, 3
    x = torch.randn(n, ldx, device=dev).to(torch.bfloat16)
    w = torch.randn(conv_dim, ck, device=dev) * 0.5
    state0 = torch.randn(slots, conv_dim, ck, device=dev)
    in_slot = torch.full((n,), 1, dtype=torch.int32, device=dev)
    parent = torch.arange(-1, n - 1, dtype=torch.int32, device=dev)
    out_slot = torch.full((n,), -1, dtype=torch.int32, device=dev)
    out_slot[-1] = 1
    sa, sb = state0.clone(), state0.clone()
    oa = torch.zeros(n, conv_dim, device=dev)
    ob = torch.zeros(n, conv_dim, device=dev)
    K.gdn_conv(x, sa, w, in_slot, parent, out_slot, oa, n, conv_dim, ck, phase=1)
    K.gdn_conv(x, sa, w, in_slot, parent, out_slot, oa, n, conv_dim, ck, phase=2)
    assert K.gdn_conv_chain(x, sb, w, in_slot, parent, out_slot, ob, n, conv_dim, ck)
    torch.cuda.synchronize()
    assert torch.equal(oa, ob)
    assert torch.equal(sa, sb)
    seq = torch.cat([state0[1].t(), x[:, :conv_dim].float()], 0)          # [ck + n, conv_dim]
    win = torch.stack([seq[i + 1:i + 1 + n] for i in range(ck)], -1)       # [n, conv_dim, ck]
    ref = torch.nn.functional.silu((win * w).sum(-1))
    assert (ob - ref).abs().max().item() < 1e-4
    assert torch.equal(sb[1], seq[-ck:].t())
    assert torch.equal(sb[0], state0[0]) and torch.equal(sb[2], state0[2])


@pytest.mark.parametrize("T", [64, 333, 2048, 4096])
def test_chunked_prefill_matches_exact_kernel(T):
    """The tensor-core chunked form against the exact recurrence: outputs, the state at a mid-chain checkpoint and at
    the end, and one decode step continued from either state, all to tf32 rounding."""
    from velogb10_b200.ops import kernels as K, lib
    torch.manual_seed(T)
    dev = "cuda"
    nk, nv, kd, vd = 2, 6, 128, 128
    key_dim, value_dim = nk * kd, nv * vd
    conv_dim = 2 * key_dim + value_dim
    ldp = (conv_dim + value_dim + 2 * nv + 7) // 8 * 8
    qkv = torch.randn(T + 1, conv_dim, device=dev)
    proj = torch.randn(T + 1, ldp, device=dev).to(torch.bfloat16)
    A_log = torch.randn(nv, device=dev) * 0.5
    dt_bias = torch.randn(nv, device=dev) * 0.5
    norm_w = torch.rand(vd, device=dev) + 0.5
    S0 = torch.randn(4, nv, kd, vd, device=dev) * 0.1
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    mid = T // 2 + 5 if T > 64 else T        # a checkpoint that is not on a chunk boundary
    off = (conv_dim, conv_dim + value_dim, conv_dim + value_dim + nv)

    # exact: one chain, state checkpointed after token mid - 1 (slot 0) and after the last token (slot 2)
    Sa = S0.clone()
    oa = torch.zeros(T, value_dim, dtype=torch.float16, device=dev)
    out_slot = [-1] * T
    out_slot[mid - 1] = 0
    out_slot[T - 1] = 2
    K.gdn_prefill(qkv, proj, *off, Sa, A_log, dt_bias, norm_w, 0, T, i32([1] * T), i32(out_slot), oa, nk, nv, kd, vd, 1e-6)

    # chunked: one call per segment between checkpoints; the second segment continues from the checkpoint slot
    Sb = S0.clone()
    ob = torch.zeros_like(oa)
    work = torch.zeros(K.gdn_chunk_work_bytes(T, nv) + 1024, dtype=torch.uint8, device=dev)
    work = work[(-work.data_ptr()) % 1024:]
    o_raw = torch.zeros(T * value_dim, device=dev)
    in_slot = i32([1] * mid + [0] * (T - mid))
    out_t = i32(out_slot)
    K.gdn_chunk_prefill(qkv, proj, *off, Sb, A_log, dt_bias, norm_w, 0, mid, in_slot, out_t, ob, nk, nv, kd, vd, 1e-6, work, o_raw)
    if mid < T:
        K.gdn_chunk_prefill(qkv, proj, *off, Sb, A_log, dt_bias, norm_w, mid, T - mid, in_slot, out_t, ob, nk, nv, kd, vd, 1e-6,
                            work, o_raw)
    torch.cuda.synchronize()
    lib.check_err_word()
    rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
    assert rel(ob, oa) < 2e-3, ("outputs", rel(ob, oa))
    assert rel(Sb[0], Sa[0]) < 1e-3, ("checkpoint state", rel(Sb[0], Sa[0]))
    assert rel(Sb[2], Sa[2]) < 1e-3, ("final state", rel(Sb[2], Sa[2]))
    assert torch.equal(Sb[1], S0[1]) and torch.equal(Sb[3], S0[3])          # untouched slots
    # one decode step from each final state (the step kernel is exact): the outputs must agree as closely
    outs = []
    for Sx in (Sa, Sb):
        o1 = torch.zeros(1, value_dim, dtype=torch.float16, device=dev)
        K.gdn_step(qkv[T:], proj[T:], *off, Sx, A_log, dt_bias, norm_w, i32([0]), i32([1]), 1, i32([2]), i32([-1]), i32([3]), o1,
                   nk, nv, kd, vd, 1e-6)
        outs.append(o1)
    torch.cuda.synchronize()
    assert rel(outs[1], outs[0]) < 2e-3


def test_step_kernel_row_quantisation_forms_agree_and_match_the_standalone_quantiser():
    """The step kernel's fused FP4-series output: the form in which every head quantises its own share (small grids,
    all CTAs resident) and the form in which the last head quantises the row (large grids) write the same bytes,
    and both equal the stand-alone quantiser run on the kernel's f16 output. Counters are left zeroed."""
    from velogb10_b200.ops import gemm as G, kernels as K, lib
    torch.manual_seed(11)
    dev = "cuda"
    nk, nv, kd, vd = 16, 48, 128, 128
    key_dim, value_dim = nk * kd, nv * vd
    conv_dim = 2 * key_dim + value_dim
    ldp = (conv_dim + value_dim + 2 * nv + 7) // 8 * 8
    n = 8                                                   # 8 chains x 48 heads > 148 CTAs: last-head form
    qkv = torch.randn(n, conv_dim, device=dev)
    proj = torch.randn(n, ldp, device=dev).to(torch.bfloat16)
    A_log = torch.randn(nv, device=dev) * 0.5
    dt_bias = torch.randn(nv, device=dev) * 0.5
    norm_w = torch.rand(vd, device=dev) + 0.5
    S0 = torch.randn(n + 1, nv, kd, vd, device=dev) * 0.1
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    kp = (value_dim + 255) // 256 * 256
    off = (conv_dim, conv_dim + value_dim, conv_dim + value_dim + nv)

    def run(cols):
        S = S0.clone()
        o = torch.zeros(n, value_dim, dtype=torch.float16, device=dev)
        bq = torch.zeros(64, kp // 2, dtype=torch.uint8, device=dev)
        sfb = torch.zeros(kp // 256 * 2048, dtype=torch.uint8, device=dev)
        g0 = torch.zeros(16, device=dev)
        ctr = torch.zeros(48, dtype=torch.int32, device=dev)
        # every column its own chain, reading slot c and writing nothing; only the first `cols` columns are launched
        K.gdn_step(qkv, proj, *off, S, A_log, dt_bias, norm_w, i32(list(range(cols))), i32([1] * cols), cols,
                   i32(list(range(n))), i32([-1] * n), i32([-1] * n), o, nk, nv, kd, vd, 1e-6, quant=(bq, sfb, g0, ctr))
        torch.cuda.synchronize()
        lib.check_err_word()
        assert int(ctr.abs().sum()) == 0
        return o, bq, sfb, g0

    o_big, bq_big, sf_big, g_big = run(n)                   # 384 CTAs
    o_small, bq_small, sf_small, g_small = run(2)           # 96 CTAs: every head quantises its share
    rows = [t * 16 + c for t in range(4) for c in range(2)]
    assert torch.equal(o_big[:2], o_small[:2])
    assert torch.equal(bq_big[rows], bq_small[rows])
    assert torch.equal(g_big[:2], g_small[:2])
    # scale bytes of columns 0..1: chunk layout [slab][step][(row & 31) * 16 + (row >> 5) * 4 + kb]
    sfv_b, sfv_s = sf_big.view(-1, 4, 32, 4, 4), sf_small.view(-1, 4, 32, 4, 4)
    for r in rows:
        assert torch.equal(sfv_b[:, :, r & 31, r >> 5], sfv_s[:, :, r & 31, r >> 5])
    # the stand-alone quantiser on the same f16 rows
    ref_bq, ref_sf, ref_g = (t.clone() for t in G.quantize_act_fp4(o_big, n, kp))
    torch.cuda.synchronize()
    allrows = [t * 16 + c for t in range(4) for c in range(n)]
    assert torch.equal(ref_bq[allrows], bq_big[allrows]) and torch.equal(ref_g[:n], g_big[:n])
