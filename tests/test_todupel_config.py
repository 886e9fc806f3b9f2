"""Todupel without a GPU: reading config.json, the plan it turns into, which tensors each layer declares, and the
plain implementation against its own token-by-token reading."""

import copy

import numpy as np
import pytest
import torch

import plain_todupel as plain
from todupel_configs import T_A, T_B, T_C, TODUPEL

from dynalm_b200.errors import Corrupt, InvalidArgument, NotFound, Unsupported
from dynalm_b200.registry import find_architecture
from dynalm_b200.weights import write_model_folder
from dynalm_b200.weights.loader import WeightMismatch, expected_tensors, open_model_folder


def _plan(cfg):
    arch = find_architecture(cfg)
    return arch.read_config(cfg), arch.plan(arch.read_config(cfg))


def test_config_reads_every_size_per_layer():
    cfg, plan = _plan(T_B)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (257, 80, 3e-5)
    m0, m1, m2 = (l.mixer for l in cfg.layers)
    assert (m0.heads, m0.kv_heads, m0.dim, m0.vdim, m0.softcap, m0.diff, m0.temp_coef, m0.temp_every) == (6, 2, 48, 16, 3.0, 0.6, 0.7, 5)
    assert (m1.heads, m1.kv_heads, m1.dim, m1.vdim, m1.scale) == (3, 1, 32, 48, 0.3)
    assert m2.kv_from == 0 and m0.kv_from is None
    assert cfg.layers[1].mlp is None and cfg.layers[2].mlp.ff == 64
    assert [r.cache_of for r in plan.order] == [None, None, 0]
    s = plan.layers[2].mixer
    assert (s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, s.scale, s.softcap, s.lambda_init, s.temp_every, s.own_kv) == \
        (6, 2, 48, 16, 0.15, 40.0, 0.55, 3, False)
    assert "ffn" not in plan.layers[1].parts and plan.layers[0].ffn.inner == 112


def test_keys_left_out_switch_a_mechanism_off():
    cfg, plan = _plan(T_C)
    m = cfg.layers[0].mixer
    assert m.softcap == 0.0 and m.temp_every == 0 and m.scale == 64 ** -0.5
    assert [r.cache_of for r in plan.order] == [None, 0, None, 2]


def test_layers_that_read_another_layers_records_declare_no_key_and_value_tensors():
    _, plan = _plan(T_A)
    names = set(expected_tensors(plan))
    assert {"l0.mix.k", "l0.mix.v", "l0.mix.k.norm", "l1.mix.k", "l2.mix.q", "l2.mix.q.norm", "l2.mix.lq1", "embed", "head",
            "final.norm", "l2.mlp.up"} <= names
    assert not {"l2.mix.k", "l2.mix.v", "l2.mix.k.norm"} & names
    shapes = {n: d.shape for n, d in expected_tensors(plan).items()}
    assert shapes["l0.mix.q"] == (4 * 2 * 16, 96) and shapes["l0.mix.k"] == (2 * 2 * 16, 96)
    assert shapes["l0.mix.v"] == (2 * 32, 96) and shapes["l0.mix.o"] == (96, 4 * 32) and shapes["l0.mix.lk2"] == (16,)


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), InvalidArgument),          # not an earlier layer
    (lambda c: c["layers"][1]["mixer"].update(kv_from=0) or c["layers"][2]["mixer"].update(kv_from=1), InvalidArgument),
    (lambda c: c["layers"][2]["mixer"].update(dim=32), Corrupt),                     # another size than its source
    (lambda c: c["layers"][0].update(type="recurrent"), Unsupported),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), Unsupported),
    (lambda c: c["layers"][0]["mixer"].pop("heads"), NotFound),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), InvalidArgument),            # 3 heads on 2 groups
    (lambda c: c.pop("layers"), NotFound),
])
def test_config_refusals(change, error):
    cfg = copy.deepcopy(T_A)
    change(cfg)
    with pytest.raises(error):
        _plan(cfg)


def test_a_folder_is_written_read_and_checked(tmp_path):
    write_model_folder(str(tmp_path), T_A, 3, dtype=torch.bfloat16)
    folder = open_model_folder(str(tmp_path))
    assert folder.architecture.name == "Todupel" and len(folder.plan.layers) == 3
    folder.close()
    # the same tensors under a configuration whose third layer has keys of its own: one error that lists them
    other = copy.deepcopy(T_A)
    other["layers"][2]["mixer"].pop("kv_from")
    import json
    (tmp_path / "config.json").write_text(json.dumps(other))
    with pytest.raises(WeightMismatch) as e:
        open_model_folder(str(tmp_path))
    assert set(e.value.missing) == {"l2.mix.k", "l2.mix.v", "l2.mix.k.norm"}


@pytest.mark.parametrize("name", sorted(TODUPEL))
def test_plain_whole_sequence_equals_plain_token_by_token(name, tmp_path):
    cfg, seed = TODUPEL[name]
    write_model_folder(str(tmp_path), cfg, seed, dtype=torch.float32)
    model = plain.PlainTodupel(str(tmp_path))
    tokens = [int(t) for t in np.random.RandomState(2).randint(0, cfg["vocab"], size=37)]
    assert np.abs(model.logits(tokens) - model.logits_stepwise(tokens)).max() < 1e-12


def test_plain_mechanisms_by_hand():
    assert np.allclose(plain.rms_norm(np.array([3.0, 4.0]), 0.0), np.array([3.0, 4.0]) / np.sqrt(12.5))
    # the temperature steps when p + 1 reaches a multiple of `every`
    t = plain.query_temperature(np.arange(12), 0.5, 4)
    assert np.allclose(t[:3], 1.0) and np.allclose(t[3:7], 1 + 0.5 * np.log(2.0)) and np.allclose(t[7:11], 1 + 0.5 * np.log(3.0))
    assert np.allclose(plain.capped(np.array([100.0, -100.0, 0.1]), 5.0), [5.0, -5.0, 5 * np.tanh(0.02)])
    w = plain.causal_softmax(np.zeros((2, 3)), np.array([0, 2]), np.arange(3))
    assert np.allclose(w, [[1, 0, 0], [1 / 3, 1 / 3, 1 / 3]])
    assert plain.diff_lambda(np.ones(2), np.zeros(2), np.ones(2), np.ones(2) * 0.5, 0.25) == pytest.approx(1 - np.e + 0.25)
    o = plain.diff_combine(np.array([[2.0, 0.0]]), np.array([[0.0, 2.0]]), 1.0, 0.25, 0.0)
    assert np.allclose(o, np.array([[1.0, -1.0]]) * 0.75)
    assert np.allclose(plain.relu2_mlp(np.array([[1.0, -2.0]]), np.eye(2), np.array([[1.0, 1.0]])), [[1.0]])


def test_split_count_of_the_single_token_kernel():
    """Every part keeps 256 keys, there are at most 32, few rows are dealt finer than many, and the count depends on the
    span only through its power of two (a growing context keeps its launch shape)."""
    from dynalm_b200.kernels.diff_attention import split_count
    for rows in (1, 3, 8, 64, 200):
        for span in (1, 17, 255, 256, 257, 2000, 5000, 70000):
            n = split_count(rows, 16, 4, span, sms=148)
            bucket = 256
            while bucket < span:
                bucket *= 2
            assert 1 <= n <= 32 and n * 256 <= max(bucket, 256)
            assert n == split_count(rows, 16, 4, bucket, sms=148)
    assert split_count(1, 16, 4, 4000, sms=148) >= split_count(64, 16, 4, 4000, sms=148) >= split_count(500, 16, 4, 4000, sms=148) == 1
    assert split_count(8, 16, 4, 100, sms=148) == 1
