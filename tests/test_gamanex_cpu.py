"""Gamanex without a GPU: the float64 restatement agrees with itself (a prefix's logits do not change when tokens follow, a borrowed cache
equals the lender's, the mechanisms do what their formulas say on hand-made inputs) and the synthetic checkpoints have the layout the
loader reads."""
import json
import math

import numpy as np
import torch

from tests import gamanex_plain as P
from uzu_b200 import safetensors_io as st
from uzu_b200 import synth

F64 = torch.float64


def small():
    return P.make_config(40, 50, [
        P.attention_layer(4, 2, 6, 10, q_temp=(0.4, 3), mlp=P.dense_mlp(24)),
        P.attention_layer(4, 2, 6, 10, scale=0.3, kv_from=0, mlp=P.moe_mlp(12, 5, 2)),
        P.attention_layer(2, 1, 8, 4, mlp=None),
    ], eps=1e-5, logit_scale=0.6)


def test_logits_of_a_prefix_do_not_depend_on_what_follows():
    cfg = small()
    w = P.random_weights(cfg, 1)
    toks = np.random.default_rng(0).integers(0, 50, 30).tolist()
    whole = P.forward(cfg, w, toks)
    for n in (1, 2, 17):
        assert torch.allclose(P.forward(cfg, w, toks[:n]), whole[:n], atol=1e-10)


def test_temperature_steps_at_multiples_of_every():
    t = P.query_temperature([0, 1, 2, 3, 4, 5, 8], 0.5, 3)
    want = [1.0, 1.0, 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(2), 1 + 0.5 * math.log(3), 1 + 0.5 * math.log(4)]
    assert torch.allclose(t, torch.tensor(want, dtype=F64))


def test_distance_bias_is_zero_on_the_diagonal_and_grows_with_the_logarithm():
    b = P.distance_bias(torch.tensor([2.0, 0.5]), torch.tensor([1.0, 3.0]), torch.tensor([0, 1, 7]))
    assert torch.allclose(b[0], torch.tensor([0.0, 2 * math.log(2), 2 * math.log(8)], dtype=F64))
    assert torch.allclose(b[1], torch.tensor([0.0, 0.5 * math.log(4), 0.5 * math.log(22)], dtype=F64))


def test_weights_are_not_normalised_over_keys():
    """Two identical visible keys give twice the output of one; a key after the query gives nothing."""
    q = torch.ones(1, 4)
    k = torch.ones(3, 4)
    v = torch.tensor([[1.0, 2.0], [1.0, 2.0], [50.0, 50.0]])
    z = torch.zeros(1)
    one = P.sigmoid_attention(q, k[:1], v[:1], [0], [0], 1, 1, 4, 2, 0.5, z, z, z)
    two = P.sigmoid_attention(q, k, v, [1], [0, 1, 2], 1, 1, 4, 2, 0.5, z, z, z)
    assert torch.allclose(two, 2 * one) and torch.allclose(one, torch.sigmoid(torch.tensor(2.0, dtype=F64)) * v[:1].to(F64))


def test_grouped_heads_read_the_key_head_of_their_group():
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.randn(5, 4 * 6, generator=g), torch.randn(5, 2 * 6, generator=g), torch.randn(5, 2 * 3, generator=g)
    r1, r2, pb = torch.rand(4, generator=g), torch.rand(4, generator=g), torch.randn(4, generator=g)
    pos = list(range(5))
    out = P.sigmoid_attention(q, k, v, pos, pos, 4, 2, 6, 3, 0.4, r1, r2, pb).reshape(5, 4, 3)
    for h in range(4):
        alone = P.sigmoid_attention(q.reshape(5, 4, 6)[:, h], k.reshape(5, 2, 6)[:, h // 2], v.reshape(5, 2, 3)[:, h // 2], pos, pos, 1, 1, 6, 3, 0.4,
                                    r1[h:h + 1], r2[h:h + 1], pb[h:h + 1])
        assert torch.allclose(out[:, h], alone)


def test_router_takes_the_lower_index_of_equal_logits_and_softmaxes_the_chosen():
    W = {"mlp.router": torch.eye(4, dtype=F64), "mlp.router.b": torch.tensor([0.0, 0.0, 1.0, 0.0], dtype=F64)}
    idx, wt = P.route(torch.tensor([[1.0, 2.0, 1.0, 0.5]], dtype=F64), W, "", 3)
    assert idx.tolist() == [[1, 2, 0]]
    e = torch.exp(torch.tensor([2.0, 2.0, 1.0], dtype=F64))
    assert torch.allclose(wt[0], e / e.sum())


def test_dense_feed_forward_squares_the_positive_part():
    W = {"mlp.up": torch.tensor([[1.0], [-1.0]]), "mlp.down": torch.tensor([[1.0, 10.0]])}
    assert P.dense_ff(torch.tensor([[3.0]], dtype=F64), W, "").tolist() == [[9.0]]
    assert P.dense_ff(torch.tensor([[-2.0]], dtype=F64), W, "").tolist() == [[40.0]]


def test_synthetic_checkpoint_layout(tmp_path):
    cfg = synth.gamanex_config(32, 40, [
        synth.gamanex_attention_layer(4, 2, 8, 6, synth.gamanex_dense_mlp(20), q_temp=(0.45, 16)),
        synth.gamanex_attention_layer(4, 2, 8, 6, synth.gamanex_moe_mlp(10, 3, 2), kv_from=0),
        synth.gamanex_attention_layer(2, 2, 4, 4, None),
    ], logit_scale=0.5)
    path = synth.write_gamanex_model(cfg, tmp_path / "m", seed=2)
    assert json.loads((path / "config.json").read_text())["architecture"] == "Gamanex"
    tensors, dtypes, _ = st.load(path / "model.safetensors")
    assert set(dtypes.values()) == {"BF16"}
    assert tensors["l0.mix.k"].shape == (16, 32) and tensors["l0.mix.v"].shape == (12, 32) and tensors["l0.mix.q"].shape == (32, 32)
    assert "l1.mix.k" not in tensors and "l1.mix.k.norm" not in tensors and "l1.mix.v" not in tensors
    assert tensors["l1.mlp.router"].shape == (3, 32) and tensors["l1.mlp.e2.down"].shape == (32, 10) and tensors["l1.rg2.b"].shape == (32,)
    assert "l2.norm2" not in tensors and "l2.ls2" not in tensors and tensors["l2.ls1"].shape == (32,)
    # the oracle runs on what the file holds
    w = {k: torch.from_numpy(synth.st_bits_to_f32(v)) for k, v in tensors.items()}
    out = P.forward(cfg, w, [1, 2, 3, 4])
    assert out.shape == (4, 40) and torch.isfinite(out).all()
    preset = synth.gamanex_preset(256, 100, blocks=2, experts=4, top=2)
    assert [L["mixer"].get("kv_from") for L in preset["layers"]] == [None, 0, None, 2]
