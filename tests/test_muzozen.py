"""Muzozen on the host side: configuration, spec, random weights, the cache's shared rows and the
model's own state, and the step function, batching and generation loop over the CPU double of the
kernels, against the plain implementation."""
import json

import numpy as np
import pytest
import torch

import ember_cpp_b200 as E
from ember_cpp_b200.config import ConfigError, MuzozenConfig, config_from_dict
from ember_cpp_b200.parts import CacheNeed, DecoderModel, StateNeed

import muzozen_util as U
import plain_muzozen as P
from conftest import run_batch
from cpu_ops import CpuOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: U.write_model(str(tmp_path_factory.mktemp(name)), U.config(name), U.SEEDS[name]) for name in U.CONFIGS}


@pytest.fixture(scope="module")
def plains(folders):
    return {name: P.PlainMuzozen(folder) for name, folder in folders.items()}


def cpu_engine(folder, max_tokens=1024, dtype="float32"):
    return E.Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, device="cpu", ops=CpuOps())


# ------------------------------------------------------------------------------ configuration
def test_the_architecture_is_registered_and_its_configuration_round_trips():
    cfg = config_from_dict(U.config("muz_a"))
    assert isinstance(cfg, MuzozenConfig) and "Muzozen" in E.config.architectures()
    assert (cfg.vocab, cfg.width, cfg.norm_eps, len(cfg.layers)) == (300, 64, 1e-5, 7)
    assert cfg.embedding == {"scale": 2.0, "bigram": {"buckets": 211, "mul_prev": 31, "mul_cur": 7}}
    assert config_from_dict(cfg.to_dict()) == cfg
    assert config_from_dict(U.config("muz_c")).embedding["bigram"] is None


@pytest.mark.parametrize("path, value, word", [
    (("width",), None, "width"), (("norm", "eps"), 0, "norm.eps"), (("layers", 0, "type"), "window", "type"),
    (("embedding", "bigram", "buckets"), 0, "buckets"), (("embedding", "scale"), "big", "scale"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 1, "mixer", "conv"), None, "conv"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mixer", "rot", "dims"), 32, "rot.dims"),
    (("layers", 2, "mixer", "kv_from"), 1, "kv_from"), (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),
    (("layers", 6, "mixer", "kv_from"), 2, "kv_from"), (("layers", 2, "mixer", "kv_rank"), 16, "kv_rank"),
    (("layers", 0, "mixer", "rot", "scaling", "factor"), None, "factor"), (("layers", 3, "mlp", "kind"), "moe", "kind")])
def test_a_bad_value_is_refused_by_its_key(path, value, word):
    d = U.config("muz_a")
    at = d
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_the_spec_follows_the_configuration():
    spec = E.config.get_architecture("Muzozen").build_spec(config_from_dict(U.config("muz_a")))
    assert [l.block for l in spec.layers] == ["shared_norm"] * 7 and spec.position.kind == "none" and spec.head == "head"
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "gated_delta_rule", "latent_attention", "gated_delta_rule"] + ["latent_attention"] * 3
    assert [a.cache_of for a in spec.schedule] == [None, None, 0, None, None, 4, 0]
    assert [None if l.ffn is None else l.ffn.params["inner"] for l in spec.layers] == [96, 96, None, 40, 72, 72, 24]
    assert all(l.norm2 is None for l in spec.layers) and spec.embedding_scale == 2.0 and spec.embed_norm.prefix == "embed.norm"
    model = DecoderModel(spec)
    names = {w.name: w.shape for w in model.weight_specs()}
    assert names["bigram"] == (212, 64) and names["embed.norm"] == (64,) and names["l0.norm1"] == (64,)
    assert names["l0.mix.dkv"] == (48, 64) and names["l0.mix.dkv.norm"] == (32,) and "l2.mix.dkv" not in names
    assert names["l0.mix.uq"] == (4 * 32, 24) and names["l5.mix.uk"] == (3 * 32, 16) and names["l6.mix.uv"] == (160, 32)
    assert names["l1.mix.q.conv"] == (32, 4) and names["l1.mix.v"] == (32, 64) and names["l3.mix.norm"] == (16,)
    assert names["l1.mlp.up"] == (96, 64) and "l2.mlp.up" not in names
    needs = model.application_needs()
    assert needs[0][0] == CacheNeed("full", 1, 32, 0, 0, 16) and needs[2][0] is None and needs[4][0] == CacheNeed("full", 1, 16, 0, 0, 16)
    assert needs[1][1] == {"S": StateNeed((4, 16, 8)), "conv": StateNeed((3, 96))}
    assert model.model_state_needs() == {"embed0.": StateNeed((1,), 0, "int32")}
    no_pairs = DecoderModel(E.config.get_architecture("Muzozen").build_spec(config_from_dict(U.config("muz_c"))))
    assert no_pairs.model_state_needs() == {} and "bigram" not in {w.name for w in no_pairs.weight_specs()}


def test_layers_that_share_rows_share_one_view_of_the_cache(folders):
    eng = cpu_engine(folders["muz_a"])
    views = eng.cache.views
    assert views[2] is views[0] and views[6] is views[0] and views[5] is views[4] and views[4] is not views[0]
    assert [a.writes_cache for a in eng.apps] == [True, False, False, False, True, False, False]
    assert len(eng.cache.groups) == 2 and list(eng.cache.model_states) == ["embed0."]


# ------------------------------------------------------------------------------ the plain implementation by itself
def test_plain_pair_rows_and_rotation():
    assert P.pair_rows([5, 9, 9], 7, 3, 2) == [7, (15 + 18) % 7, (27 + 18) % 7]
    cos, sin = P.rotation_tables({"dims": 4, "base": 100.0, "scaling": None}, 3)
    assert np.allclose(cos[2], [np.cos(2.0), np.cos(0.2)]) and np.allclose(sin[1], [np.sin(1.0), np.sin(0.1)])
    x = np.arange(12.0).reshape(2, 1, 6)
    y = P.rotate(x, cos, sin, 4)
    assert np.allclose(y[0], x[0]) and np.allclose(y[1, 0, 4:], x[1, 0, 4:])        # position 0 and the dimensions past `dims`
    assert np.allclose(y[1, 0, 0], 6 * np.cos(1.0) - 8 * np.sin(1.0)) and np.allclose(y[1, 0, 3], 9 * np.cos(0.1) + 7 * np.sin(0.1))
    scaled_cos, _ = P.rotation_tables({"dims": 16, "base": 10000.0, "scaling": U.YARN_A}, 2)
    plain_cos, _ = P.rotation_tables({"dims": 16, "base": 10000.0, "scaling": None}, 2)
    mag = 0.1 * np.log(8.0) + 1.0
    assert np.allclose(scaled_cos[1, 0], plain_cos[1, 0] * mag)                      # the fastest pair keeps its frequency
    assert np.allclose(scaled_cos[1, -1], np.cos(10000.0 ** (-14 / 16) / 8.0) * mag)  # the slowest one is stretched


def test_plain_delta_rule_overwrites_what_a_key_holds():
    """With beta = 1 and no decay, writing (k, v2) after (k, v1) leaves v2 under k: the rule corrects, it does not add."""
    k = np.array([[1.0, 0.0], [1.0, 0.0], [0.0, 1.0]])
    v = np.array([[3.0], [5.0], [7.0]])
    out = P.delta_recurrence(k, k, v, np.ones(3), np.ones(3))
    assert np.allclose(out[:, 0], [3.0, 5.0, 7.0])
    out = P.delta_recurrence(np.array([[1.0, 0.0]] * 3), k, v, np.ones(3), np.array([1.0, 1.0, 0.5]))
    assert np.allclose(out[:, 0], [3.0, 5.0, 2.5])


def test_plain_state_matters(plains):
    m = plains["muz_a"]
    seq = U.ids(5, 300, 30)
    whole = P.forward(m, seq)
    assert U.row_error(P.forward(m, seq[20:])[-1], whole[-1]) > 1e-3


# ------------------------------------------------------------------------------ the step function over the CPU double
@pytest.mark.parametrize("name", ["muz_a", "muz_b", "muz_c", "muz_d", "muz_e"])
def test_steps_equal_whole_sequences(folders, plains, name):
    """Whole prompts, one token at a time from the first token on, portions down to two tokens, and unequal
    batches decoded together: all give the plain implementation's logits at every position."""
    eng, m = cpu_engine(folders[name]), plains[name]
    vocab = m.cfg["vocab"]
    seqs = [U.ids(10 + i, vocab, n) for i, n in enumerate((130, 1, 40, 70))]
    refs = [P.forward(m, s) for s in seqs]
    got, _ = run_batch(eng, seqs, [len(s) for s in seqs])
    assert max(U.row_error(g, r) for g, r in zip(got, refs)) < 1e-5
    got, _ = run_batch(eng, seqs, [100, 1, 1, 30])                         # prompts, then one token each
    assert max(U.row_error(g, r) for g, r in zip(got, refs)) < 1e-5
    slot, at, rows = eng.open(), 0, []
    for n in (2, 5, 64, 3, 2, 30, 24):                                     # portions of one sequence
        rows.append(eng.step([(slot, seqs[0][at:at + n], list(range(n)))]).numpy())
        at += n
    eng.close(slot)
    assert U.row_error(np.concatenate(rows), refs[0]) < 1e-5
    eng.cache.check()
    assert eng.cache.slots.held == 0 and all(g.pages.held == 0 for g in eng.cache.groups)


def test_the_stream_after_every_layer(folders, plains):
    """The residual stream itself, layer by layer, not only the logits (taken with a hook on the blocks)."""
    eng, m = cpu_engine(folders["muz_b"]), plains["muz_b"]
    seq = U.ids(3, 200, 21)
    _, streams = P.forward(m, seq, return_layers=True)
    seen = []
    for block in eng.model.blocks:
        inner = block.forward

        def hooked(ctx, x, app, inner=inner):
            out = inner(ctx, x, app)
            seen.append(out.clone())          # (a copy: the next layer adds into the stream in place)
            return out
        block.forward = hooked
    slot = eng.open()
    eng.step([(slot, seq, [])])
    assert len(seen) == len(streams)
    for got, want in zip(seen, streams):
        assert np.abs(got.numpy() - want).max() < 1e-4 * np.abs(want).max()


def test_slots_and_pages_that_are_used_again_carry_nothing_over(folders, plains):
    eng, m = cpu_engine(folders["muz_a"], max_tokens=256), plains["muz_a"]
    for round_ in range(3):
        seqs = [U.ids(100 * round_ + i, 300, n) for i, n in enumerate((70, 90))]
        got, slots = run_batch(eng, seqs, [60, 2])
        assert sorted(slots) == [0, 1]
        assert max(U.row_error(g, P.forward(m, s)) for g, s in zip(got, seqs)) < 1e-5


def test_greedy_generation_through_the_session(folders, plains):
    for name in ("muz_a", "muz_b"):
        m = plains[name]
        session = E.Session(folders[name], None, max_batch_size=3, dtype="float32", max_tokens=1024, ops=CpuOps(), device="cpu")
        prompts = [U.ids(50 + i, m.cfg["vocab"], n) for i, n in enumerate((5, 23, 1, 9))]
        out = session.generate_batch(prompts, steps=6, temperature=0.0)
        assert out == [P.generate(m, p, 6) for p in prompts]


def test_the_command_line_writes_a_random_model_of_this_design(tmp_path):
    from ember_cpp_b200 import cli
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(U.config("muz_b")))
    out = tmp_path / "model"
    assert cli.main([str(out), "-", "1", "random-weights", "--config", str(cfg_file), "--seed", "5"]) == 0
    cfg = E.load_config(str(out))
    assert isinstance(cfg, MuzozenConfig) and cfg.width == 96
    eng = cpu_engine(str(out), max_tokens=128)
    slot = eng.open()
    logits = eng.step([(slot, U.ids(1, 200, 9), [8])])
    assert tuple(logits.shape) == (1, 200) and bool(torch.isfinite(logits).all())
