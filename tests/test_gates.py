"""Gate functions on the CPU oracle and the statistics of the gate runner."""
import json

from velogb10_b200 import gate, gates
from velogb10_b200.checkpoint.synthetic import SyntheticSource
from velogb10_b200.config import tiny_hybrid
from velogb10_b200.models.oracle import OracleModel
from velogb10_b200.models.weights import ModelBuilder


def _runner():
    cfg = tiny_hybrid(mtp=True)
    w = ModelBuilder(cfg, SyntheticSource(cfg, 0, std=0.08), recipe="all").build()
    r = OracleModel(w)
    r.alloc_state(4, 4 + 17 + 4, 320)
    return r, cfg


def test_gates_pass_on_oracle(capsys):
    r, cfg = _runner()
    assert gates.gate_verify_fuzz(r, cfg, draws=2, seed=1, max_seq=300) == 0
    assert gates.gate_state(r, cfg) == 0
    assert gates.gate_tree(r, cfg) == 0
    assert gates.gate_lanes(r, cfg) == 0
    assert gates.gate_mtp_lossless(r, cfg, n_new=12, depth=3) == 0
    assert gates.dump_argmax(r, cfg, 6) == 0
    assert gates.perplexity(r, cfg, 12) == 0
    out = capsys.readouterr().out
    assert "GATE_TOKENS" in out and '"LOSSLESS_OK": true' in out
    tab = gates.calibrate_mtp_r(r, steps=1)
    assert set(tab) == {2, 3, 4, 5, 6, 8} and all(v > 0 for v in tab.values())


def test_negative_control_trips_the_verify_gate(capsys):
    """A runner whose verify path differs from its decode path must fail the gate (the detector trips)."""
    r, cfg = _runner()
    real = r.verify

    def broken(slot, tokens, pos_start, ckpt_base=None, parent=None):
        lg, h = real(slot, tokens, pos_start, ckpt_base, parent)
        lg = lg.clone()
        lg[-1, 0] += 1e-3
        return lg, h

    r.verify = broken
    assert gates.gate_verify_fuzz(r, cfg, draws=1, seed=0, max_seq=300) == 1


def test_statistics():
    assert abs(gates.wh_z(10.0, 10)) < 0.2 and gates.wh_z(40.0, 10) > 4
    a = {i: 100 for i in range(10)}
    chi2, dof = gates.two_sample_chi2(a, dict(a))
    assert chi2 == 0 and dof == 9
    b = dict(a); b[0] = 300
    assert gates.wh_z(*gates.two_sample_chi2(a, b)) > 4
    lo, hi = gate.sprt_bounds()
    assert lo < 0 < hi
    verdict, n = gate.sprt(lambda i: True)
    assert verdict == "pass" and 10 <= n <= 20
    assert gate.sprt(lambda i: False)[0] == "fail"
    assert gate.sprt(lambda i: None)[0] == "unmeasured"
    hist = [100, 101, 99, 100, 102, 98, 100, 101]
    assert gate.shewhart_cusum(hist, 100.5)["status"] == "ok"
    assert gate.shewhart_cusum(hist, 80.0)["status"] == "drift"
    assert gate.shewhart_cusum(hist[:3], 100.0)["status"] == "collecting"
    try:
        gate.extract(json.dumps({"a": 1}), "tok_s")
        raise AssertionError("missing key must raise")
    except KeyError:
        pass
