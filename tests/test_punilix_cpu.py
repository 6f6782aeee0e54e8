"""CPU-side checks of the Punilix support: the plain restatement is consistent with itself (prompt vs steps), the synthetic checkpoints
have the layout the loader reads, and the trace runner speaks its line protocol (engine replaced by a recorder: no GPU here)."""
import io
import json
import math
import sys

import numpy as np
import torch

from tests import punilix_plain as P
from uzu_b200 import safetensors_io as st
from uzu_b200 import synth


def small_config():
    S = synth
    return S.punilix_config(48, 90, [
        S.punilix_delta_layer(2, 12, S.punilix_dense_mlp(20, limit=1.0)),
        S.punilix_latent_layer(3, 8, 4, 10, 12, 14, S.punilix_moe_mlp(8, 5, 2), scaling={"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}),
    ], norm_groups=2, logit_softcap=8.0)


def oracle(cfg, seed=0):
    return P.PlainModel(cfg, {k: torch.from_numpy(np.asarray(v)) for k, v in synth.punilix_tensors(cfg, seed).items()})


def test_plain_model_steps_equal_the_whole_prompt():
    cfg = small_config()
    m = oracle(cfg)
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 30).tolist()
    whole = m.step(toks)
    m.reset()
    parts = torch.cat([m.step(toks[:7]), m.step(toks[7:9]), *[m.step([t]) for t in toks[9:]]])
    assert (whole - parts).abs().max() < 1e-9
    assert whole.abs().max() <= 8.0          # soft cap


def test_rotary_frequencies_blend():
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, mult = P.rotary_frequencies(rot)
    assert math.isclose(mult, 0.1 * math.log(4.0) + 1.0)
    where = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(where(8.0)), 0), min(math.ceil(where(1.0)), 7)
    for i in range(4):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        plain = 100.0 ** (-2.0 * i / 8)
        assert math.isclose(float(f[i]), plain / 4.0 * ramp + plain * (1 - ramp), rel_tol=1e-12)
    g, one = P.rotary_frequencies({"dims": 8, "base": 100.0, "scaling": None})
    assert one == 1.0 and math.isclose(float(g[1]), 100.0 ** -0.25)


def test_delta_rule_replaces_along_a_repeated_key():
    """decay 1, rate 1: writing twice along the same unit key leaves only the second value there."""
    dim = 6
    p = {n: torch.zeros(dim, dim, dtype=P.F64) for n in ("r", "k", "v", "g", "a", "o")}
    p.update({"w1": torch.zeros(2, dim, dtype=P.F64), "w2": torch.zeros(dim, 2, dtype=P.F64), "w0": torch.full((dim,), -60.0, dtype=P.F64),
              "a.b": torch.full((dim,), 60.0, dtype=P.F64), "norm": torch.ones(dim, dtype=P.F64)})
    p["k"][0, 0] = 1.0; p["r"][0, 0] = 1.0          # key = read = first input coordinate, along channel 0
    p["v"] = torch.eye(dim, dtype=P.F64)
    p["o"] = torch.eye(dim, dtype=P.F64)
    state = torch.zeros(1, dim, dim, dtype=P.F64)
    h = torch.tensor([[1.0, 0, 2, 0, 0, 0], [1.0, 0, 0, 3, 0, 0]], dtype=P.F64)
    P.general_delta(h, p, 1, dim, 1e-6, state)
    assert torch.allclose(state[0][0], h[1], atol=1e-5)      # row 0 of the state holds the second value only


def test_synthetic_checkpoint_layout(tmp_path):
    cfg = small_config()
    path = synth.write_punilix_model(cfg, tmp_path / "m", seed=3)
    assert json.loads((path / "config.json").read_text())["architecture"] == "Punilix"
    tensors, dtypes, _ = st.load(path / "model.safetensors")
    assert dtypes["embed"] == "BF16" and tensors["embed"].shape == (90, 48)
    assert dtypes["l1.mlp.table"] == "I32" and tensors["l1.mlp.table"].shape == (90, 2)
    assert all(len(set(row)) == 2 for row in tensors["l1.mlp.table"].tolist())
    assert tensors["l1.mix.dkv"].shape == (12 + 4, 48) and tensors["l0.mix.w2"].shape[0] == 24
    assert "l0.mlp.gate" in tensors and "l1.mlp.e4.down" in tensors and "l1.mlp.gate" not in tensors


def test_trace_runner_protocol(tmp_path, monkeypatch, capsys):
    from uzu_b200 import binding, trace_runner

    calls = []

    class FakeEngine:
        def __init__(self, ctx, model, **kw):
            calls.append(("engine", kw))
            self.free, self.next = [], 0

        def slot_acquire(self):
            s = self.free.pop() if self.free else self.next
            self.next += s == self.next
            calls.append(("acquire", s))
            return s

        def slot_release(self, s):
            self.free.append(s)
            calls.append(("release", s))

        def forward_rows(self, tokens, rows, slot):
            calls.append(("rows", slot, list(tokens), list(rows)))
            return np.full((len(rows), 5), float(slot), np.float32)

        def close(self):
            pass

    class FakeContext:
        def __init__(self, device):
            pass

        def close(self):
            pass

    monkeypatch.setattr(trace_runner, "ensure_library", lambda: None)
    monkeypatch.setattr(binding, "Context", FakeContext)
    monkeypatch.setattr(binding, "Engine", FakeEngine)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [0, 2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": []}], "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": [9, 9], "want": [1]}], "end": ["b"]}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    assert trace_runner.main(["--model", "x", "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "100"]) == 0
    assert capsys.readouterr().out.split() == ["done", "0", "done", "1", "done", "2"]
    assert calls[0][1]["storage_f32"] is True and calls[0][1]["max_context_length"] == 100
    assert np.fromfile(tmp_path / "o" / "0.f32", "<f4").shape == (10,) and not (tmp_path / "o" / "1.f32").exists()
    assert np.fromfile(tmp_path / "o" / "2.f32", "<f4").shape == (5,)
    assert [c for c in calls if c[0] in ("acquire", "release")] == [("acquire", 0), ("release", 0), ("acquire", 0), ("release", 0)]
