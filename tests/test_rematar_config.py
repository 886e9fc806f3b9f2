"""Rematar without a GPU: reading config.json, the plan it turns into, which tensors each layer declares, the run
order of layers that share tensors, and the plain implementation against its own reading in portions and by hand."""

import copy
import json

import numpy as np
import pytest
import torch

import plain_rematar as plain
from rematar_configs import R_A, R_B, R_C, REMATAR

from dynalm_b200.errors import Corrupt, InvalidArgument, NotFound, Unsupported
from dynalm_b200.registry import find_architecture
from dynalm_b200.weights import write_model_folder
from dynalm_b200.weights.loader import WeightMismatch, expected_tensors, open_model_folder


def _plan(cfg, present=None):
    arch = find_architecture(cfg)
    return arch.read_config(cfg), arch.plan(arch.read_config(cfg), present)


def test_config_reads_every_size_per_layer():
    cfg, plan = _plan(R_B)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.alpha, cfg.embedding_scale) == (257, 100, 3e-5, 1.0, 1.0)
    s, a, _ = (l.mixer for l in cfg.layers)
    assert (s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups) == (5, 20, 12, 1, 2, 1)
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.q_rank, a.kv_rank, a.scale, a.window, a.rot_base, a.rot_dims) == \
        (3, 20, 12, 28, 36, 44, 9.0, 7, 500.0, 8)
    assert cfg.layers[1].mlp is None and cfg.layers[0].mlp.ff == 172
    m = plan.layers[1].mixer
    assert (m.kind, m.num_heads, m.head_dim, m.rot_dim, m.value_dim, m.kv_rank, m.window) == ("latent_attention", 3, 20, 12, 28, 44, 7)
    assert (m.position.kind, m.position.rotary_dim, m.position.theta) == ("rotary_interleaved", 8, 500.0)
    assert plan.layers[0].mixer.kind == "ssd" and plan.layers[0].mixer.taps == 2
    assert "ffn" not in plan.layers[1].parts and plan.layers[0].ffn.activation == "gelu_tanh"
    assert plan.embedding.scale == 1.0 and plan.layers[0].mixer_norm.alpha == 1.0


def test_layers_that_share_tensors_are_one_block_run_again_with_a_state_of_its_own():
    cfg, plan = _plan(R_C)
    assert [l.weights_of for l in cfg.layers] == [None, None, None, None, 0, 0]          # the chain 5 -> 4 -> 0 resolved
    assert len(plan.layers) == 4 and [r.layer for r in plan.order] == [0, 1, 2, 3, 0, 0]
    assert all(r.cache_of is None for r in plan.order)
    names = set(expected_tensors(plan))
    assert not any(n.startswith(("l4.", "l5.")) for n in names)
    cfg, plan = _plan(R_A)
    assert [r.layer for r in plan.order] == [0, 1, 1, 0] and (cfg.alpha, cfg.embedding_scale) == (2.0, 4.0)
    assert plan.layers[0].mixer_norm.alpha == 2.0 and plan.embedding.scale == 4.0


def test_keys_left_out_switch_a_mechanism_off():
    cfg, plan = _plan(R_C)
    assert cfg.layers[2].mixer.window == 0 and cfg.layers[1].mixer.window == 500
    assert cfg.layers[3].mixer.rot_dims == 0 and plan.layers[3].mixer.position is None
    assert plan.layers[2].mixer.window == 0


def test_declared_tensors_and_their_shapes():
    _, plan = _plan(R_A)
    shapes = {n: d.shape for n, d in expected_tensors(plan).items()}
    assert shapes["l1.mix.in"] == (2 * 96 + 2 * 3 * 24 + 6, 96) and shapes["l1.mix.conv"] == (96 + 144, 3)
    assert shapes["l1.mix.conv.b"] == (240,) and shapes["l1.mix.A_log"] == (6,) and shapes["l1.mix.norm"] == (96,)
    assert shapes["l1.mix.o"] == (96, 96)
    assert shapes["l0.mix.dq"] == (40, 96) and shapes["l0.mix.uq"] == (4 * 24, 40) and shapes["l0.mix.dkv"] == (56, 96)
    assert shapes["l0.mix.uk"] == (64, 48) and shapes["l0.mix.uv"] == (96, 48) and shapes["l0.mix.g"] == (96, 96)
    assert shapes["l0.mix.sink"] == (4,) and shapes["l0.ls1"] == (96,) and shapes["l0.norm2"] == (96,)
    assert {"embed", "head", "final.norm", "l0.mlp.up", "l1.mlp.down"} <= set(shapes)
    # what a file does not carry is not asked for: scales, sinks and the gate go by presence
    base = set(shapes) - {"l0.ls1", "l0.ls2", "l0.mix.sink", "l0.mix.g"}
    _, lean = _plan(R_A, present=base)
    assert set(expected_tensors(lean)) == base


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][2].update(weights_of=2), InvalidArgument),                 # not an earlier layer
    (lambda c: c["layers"][2].update(weights_of=0), Corrupt),                         # another kind than its source
    (lambda c: c["layers"][2].update(mixer=dict(c["layers"][2]["mixer"], state=8)), Corrupt),                     # another size than its source
    (lambda c: c["layers"][0].update(type="attention"), Unsupported),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), Unsupported),
    (lambda c: c["layers"][0]["mixer"].pop("heads"), NotFound),
    (lambda c: c["layers"][1]["mixer"].update(groups=4), InvalidArgument),            # 6 heads on 4 groups
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), InvalidArgument),       # 96 channels in 5 parts
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), InvalidArgument),      # more than the rotated piece
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=3), InvalidArgument),       # pairs
    (lambda c: c.pop("layers"), NotFound),
])
def test_config_refusals(change, error):
    cfg = copy.deepcopy(R_A)
    change(cfg)
    with pytest.raises(error):
        _plan(cfg)


def test_a_folder_is_written_read_and_checked(tmp_path):
    write_model_folder(str(tmp_path), R_A, 3, dtype=torch.bfloat16)
    folder = open_model_folder(str(tmp_path))
    assert folder.architecture.name == "Rematar" and len(folder.plan.layers) == 2 and len(folder.plan.order) == 4
    folder.close()
    # the same tensors under a configuration whose third layer has tensors of its own: one error that lists them
    other = copy.deepcopy(R_A)
    other["layers"][2].pop("weights_of")
    (tmp_path / "config.json").write_text(json.dumps(other))
    with pytest.raises(WeightMismatch) as e:
        open_model_folder(str(tmp_path))
    assert {"l2.mix.in", "l2.mix.conv", "l2.norm1", "l2.mlp.up"} <= set(e.value.missing)
    assert all(n.startswith("l2.") for n in e.value.missing)


@pytest.mark.parametrize("name", sorted(REMATAR))
def test_plain_whole_sequence_equals_plain_in_portions(name, tmp_path):
    cfg, seed = REMATAR[name]
    write_model_folder(str(tmp_path), cfg, seed, dtype=torch.float32)
    model = plain.PlainRematar(str(tmp_path))
    tokens = [int(t) for t in np.random.RandomState(2).randint(0, cfg["vocab"], size=45)]
    whole = model.logits(tokens)
    assert np.abs(whole - model.logits_stepwise(tokens)).max() < 1e-12
    assert np.abs(whole - model.logits_stepwise(tokens, [2, 1, 17, 3, 22])).max() < 1e-12


def test_plain_mechanisms_by_hand():
    assert np.allclose(plain.rms_norm(np.array([3.0, 4.0]), 0.0), np.array([3.0, 4.0]) / np.sqrt(12.5))
    assert np.allclose(plain.sum_then_norm(np.array([[1.0, 0.0]]), np.array([[0.0, 2.0]]), 3.0, 0.0, np.array([1.0, 2.0]),
                                           np.array([1.0, 0.5])), np.array([[3.0, 2.0]]) / np.sqrt(5.0))
    assert plain.gelu_tanh(np.array([0.0]))[0] == 0.0 and plain.gelu_tanh(np.array([10.0]))[0] == pytest.approx(10.0)
    assert plain.gelu_tanh(np.array([1.0]))[0] == pytest.approx(0.841192, abs=1e-6)
    # the last tap is the current token's; zeros stand before the start; kept inputs stand in for them later
    u = np.array([[1.0], [2.0], [4.0]])
    taps, bias = np.array([[100.0, 10.0, 1.0]]), np.array([0.5])
    assert np.allclose(plain.causal_conv(u, taps, bias)[:, 0], [1.5, 12.5, 124.5])
    assert np.allclose(plain.causal_conv(u[2:], taps, bias, before=u[:2])[:, 0], [124.5])
    # one head, one state row, one channel: S <- e^(-dt) S + dt B x, y = S C + D x
    y, S = plain.ssm_scan(np.array([[[2.0]], [[0.0]]]), np.array([[1.0], [1.0]]), np.array([[[3.0]], [[3.0]]]),
                          np.array([[[5.0]], [[5.0]]]), np.array([0.0]), np.array([7.0]))
    assert np.allclose(y[:, 0, 0], [6.0 * 5 + 14.0, 6.0 * np.exp(-1.0) * 5]) and S[0, 0, 0] == pytest.approx(6.0 * np.exp(-1.0))
    # the gate comes before the norm, every part has its own root mean square
    g = plain.gated_group_norm(np.array([[1.0, 1.0, 10.0, 10.0]]), np.full((1, 4), 50.0), 2, 0.0, np.ones(4))
    assert np.allclose(g, 1.0)
    # pair (2i, 2i + 1) turns by position * base^(-2i / dims); what lies behind `dims` passes
    v = np.array([[1.0, 0.0, 1.0, 0.0, 9.0]])
    r = plain.rotate_pairs(v, np.array([2]), 4, 100.0)
    assert np.allclose(r[0], [np.cos(2.0), np.sin(2.0), np.cos(0.2), np.sin(0.2), 9.0])
    # a window of 2 sees itself and one token back; the sink counts once in the denominator and has no value
    w = plain.window_sink_softmax(np.zeros((2, 3)), np.array([0, 2]), np.arange(3), 2, 0.0)
    assert np.allclose(w, [[0.5, 0, 0], [0, 1 / 3, 1 / 3]])
    w = plain.window_sink_softmax(np.zeros((1, 3)), np.array([2]), np.arange(3), 0, None)
    assert np.allclose(w, 1 / 3)
