"""Kernels write only what they own. Outputs, states and scratch areas are carved out of larger buffers whose
surroundings hold a poison pattern; after each kernel the surroundings must be untouched (the check a memory checker
would do, for the buffers a kernel is handed), and a second run must reproduce the first bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu

PAD = 4096
POISON = 0xA5


class Guarded:
    """A tensor of ``shape`` / ``dtype`` between two poisoned bands of ``PAD`` bytes."""

    def __init__(self, shape, dtype, fill=0):
        n = 1
        for d in shape:
            n *= d
        self.nbytes = n * torch.empty((), dtype=dtype).element_size()
        self.raw = torch.full((PAD + 1024 + self.nbytes + PAD,), POISON, dtype=torch.uint8, device="cuda")
        self.start = PAD + (-(self.raw.data_ptr() + PAD)) % 1024          # the buffer itself starts 1024-byte aligned
        self.t = self.raw[self.start:self.start + self.nbytes].view(dtype).view(shape)
        self.t.fill_(fill)

    def check(self, what):
        torch.cuda.synchronize()
        lo, hi = self.raw[:self.start], self.raw[self.start + self.nbytes:]
        assert bool((lo == POISON).all()), f"{what}: bytes before the buffer were written"
        assert bool((hi == POISON).all()), f"{what}: bytes after the buffer were written"


def _q(m, k, seed=0):
    from velogb10_b200.models.weights import QLinear
    g = torch.Generator(device="cuda").manual_seed(seed)
    return QLinear.from_dense((torch.randn(m, k, generator=g, device="cuda") * 0.05).to(torch.bfloat16), "nvfp4")


@pytest.mark.parametrize("m,k,n", [(1552, 256, 3), (5120, 6144, 1), (640, 2176, 16), (76032, 512, 5)])
def test_fp4_gemm_writes_only_its_rows(m, k, n):
    from velogb10_b200.ops import gemm as G, lib
    q = _q(m, k)
    x = torch.randn(16, k, device="cuda").to(torch.float16)
    for dt in (torch.bfloat16, torch.float32):
        out = Guarded((n, m), dt)
        G.linear_fp4(q, x, n, out=out.t)
        out.check(f"linear_fp4 {m}x{k} n={n} {dt}")
        first = out.t.clone()
        G.linear_fp4(q, x, n, out=out.t)
        torch.cuda.synchronize()
        assert torch.equal(first, out.t)
    lib.check_err_word()


@pytest.mark.parametrize("h,n", [(5120, 1), (2048, 16), (256, 5)])
def test_norm_quantiser_writes_only_its_rows(h, n):
    from velogb10_b200.ops import gemm as G, kernels as K
    res = Guarded((n, h), torch.bfloat16)
    res.t.copy_((torch.randn(n, h, device="cuda") * 2).to(torch.bfloat16))
    x16 = Guarded((n, h), torch.float16)
    delta = torch.randn(n, h, device="cuda").to(torch.bfloat16)
    w = torch.randn(h, device="cuda") * 0.1
    G.add_rmsnorm_fp4(res.t, delta, w, 1e-6, n, out16=x16.t)
    res.check("add_rmsnorm_fp4 residual")
    x16.check("add_rmsnorm_fp4 f16 output")
    res2 = Guarded((n, h), torch.bfloat16)
    res2.t.copy_(res.t)
    y16 = Guarded((n, h), torch.float16)
    K.add_rmsnorm(res2.t, delta, w, 1e-6, n, out16=y16.t)
    res2.check("add_rmsnorm residual")
    y16.check("add_rmsnorm f16 output")


@pytest.mark.parametrize("lens", [[1, 63, 700], [4096, 129], [20000]])
def test_decode_attention_stays_inside_scratch_and_output(lens):
    from velogb10_b200.ops import kernels as K, lib
    nh, nkv, hd = 24, 4, 256
    n, max_seq = len(lens), max(lens) + 8
    kc = torch.randn(n, nkv, max_seq, hd, device="cuda").to(torch.bfloat16)
    vc = torch.randn(n, nkv, max_seq, hd, device="cuda").to(torch.bfloat16)
    q = torch.randn(16, nh * hd, device="cuda").to(torch.bfloat16)
    lens_t = torch.zeros(16, dtype=torch.int32, device="cuda")
    lens_t[:n] = torch.tensor(lens, dtype=torch.int32)
    slots = torch.arange(16, dtype=torch.int32, device="cuda") % n
    for name, fn in (("tensor-core", K.attn_decode_tc), ("cuda-core", K.attn_decode)):
        part = Guarded((K.attn_scratch_floats(n, nh, hd, 32),), torch.float32)
        out = Guarded((n, nh * hd), torch.float16)
        fn(q, kc, vc, lens_t, slots, part.t, out.t, n, nh, nkv, hd)
        part.check(f"{name} decode attention partials")
        out.check(f"{name} decode attention output")
        first = out.t.clone()
        fn(q, kc, vc, lens_t, slots, part.t, out.t, n, nh, nkv, hd)
        torch.cuda.synchronize()
        assert torch.equal(first, out.t), name
    lib.check_err_word()


def test_gdn_step_stays_inside_state_and_outputs():
    from velogb10_b200.ops import kernels as K, lib
    torch.manual_seed(2)
    nk, nv, kd, vd = 4, 8, 128, 128
    key_dim, value_dim = nk * kd, nv * vd
    conv_dim = 2 * key_dim + value_dim
    ldp = (conv_dim + value_dim + 2 * nv + 7) // 8 * 8
    n, slots = 5, 7
    qkv = torch.randn(n, conv_dim, device="cuda")
    proj = torch.randn(n, ldp, device="cuda").to(torch.bfloat16)
    A_log, dt_bias = torch.randn(nv, device="cuda") * 0.5, torch.randn(nv, device="cuda") * 0.5
    norm_w = torch.rand(vd, device="cuda") + 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    S = Guarded((slots, nv, kd, vd), torch.float32)
    S.t.copy_(torch.randn(slots, nv, kd, vd, device="cuda") * 0.1)
    out = Guarded((n, value_dim), torch.float16)
    kp = (value_dim + 255) // 256 * 256
    bq = Guarded((64, kp // 2), torch.uint8)
    sfb = Guarded((kp // 256, 2048), torch.uint8)
    g0 = Guarded((16,), torch.float32)
    ctr = Guarded((48,), torch.int32)
    # one chain of five columns: reads slot 0, checkpoints into slots 2..5, final state to the last slot
    K.gdn_step(qkv, proj, conv_dim, conv_dim + value_dim, conv_dim + value_dim + nv, S.t, A_log, dt_bias, norm_w,
               i32([0]), i32([n]), 1, i32([0] * n), i32([-1, 0, 1, 2, 3]), i32([2, 3, 4, 5, slots - 1]), out.t, nk, nv, kd, vd,
               1e-6, quant=(bq.t, sfb.t, g0.t, ctr.t))
    for g, what in ((S, "state"), (out, "outputs"), (bq, "series terms"), (sfb, "series scales"), (g0, "row scales"), (ctr, "counters")):
        g.check(f"gdn_step {what}")
    assert int(ctr.t.abs().sum()) == 0
    lib.check_err_word()


def test_chunked_gdn_prefill_stays_inside_work_area_and_state():
    from velogb10_b200.ops import kernels as K, lib
    torch.manual_seed(4)
    nk, nv, kd, vd = 2, 4, 128, 128
    key_dim, value_dim = nk * kd, nv * vd
    conv_dim = 2 * key_dim + value_dim
    ldp = (conv_dim + value_dim + 2 * nv + 7) // 8 * 8
    T = 333
    qkv = torch.randn(T, conv_dim, device="cuda")
    proj = torch.randn(T, ldp, device="cuda").to(torch.bfloat16)
    A_log, dt_bias = torch.randn(nv, device="cuda") * 0.5, torch.randn(nv, device="cuda") * 0.5
    norm_w = torch.rand(vd, device="cuda") + 0.5
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    S = Guarded((3, nv, kd, vd), torch.float32)
    S.t.copy_(torch.randn(3, nv, kd, vd, device="cuda") * 0.1)
    out = Guarded((T, value_dim), torch.float16)
    work = Guarded((K.gdn_chunk_work_bytes(T, nv),), torch.uint8)
    o_raw = Guarded((T * nv * vd,), torch.float32)
    K.gdn_chunk_prefill(qkv, proj, conv_dim, conv_dim + value_dim, conv_dim + value_dim + nv, S.t, A_log, dt_bias, norm_w,
                        0, T, i32([1] * T), i32([-1] * (T - 1) + [2]), out.t, nk, nv, kd, vd, 1e-6, work.t, o_raw.t)
    for g, what in ((S, "state"), (out, "outputs"), (work, "work area"), (o_raw, "raw outputs")):
        g.check(f"gdn_chunk_prefill {what}")
    lib.check_err_word()
