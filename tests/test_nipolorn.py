"""Nipolorn on the host side: configuration, spec, random weights, the cache's kept first pages and
state rows, and the step function, batching and generation loop over the CPU double of the kernels,
against the plain implementation."""
import json
import os

import numpy as np
import pytest
import torch

import ember_cpp_b200 as E
from ember_cpp_b200.cache.sequence_cache import PAGE, SequenceCache
from ember_cpp_b200.config import ConfigError, NipolornConfig, config_from_dict
from ember_cpp_b200.parts import CacheNeed, DecoderModel, StateNeed
from ember_cpp_b200.weights import read_folder

import nipolorn_util as U
import plain_nipolorn as P
from conftest import run_batch
from cpu_ops import CpuOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: U.write_model(str(tmp_path_factory.mktemp(name)), U.config(name), U.SEEDS[name]) for name in U.CONFIGS}


@pytest.fixture(scope="module")
def plains(folders):
    return {name: P.PlainNipolorn(folder) for name, folder in folders.items()}


def cpu_engine(folder, max_tokens=1024, dtype="float32"):
    return E.Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, device="cpu", ops=CpuOps())


# ------------------------------------------------------------------------------ configuration
def test_the_architecture_is_named_by_one_string_and_registered():
    cfg = config_from_dict(U.config("nip_a"))
    assert isinstance(cfg, NipolornConfig) and "Nipolorn" in E.config.architectures()
    assert (cfg.vocab, cfg.width, cfg.norm_eps, len(cfg.layers)) == (300, 64, 1e-5, 4)
    assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("path, value, word", [
    (("width",), None, "width"), (("norm", "eps"), 0, "norm.eps"), (("layers", 0, "type"), "serial", "type"),
    (("layers", 1, "mixer", "left", "mask", "size"), 0, "mask.size"), (("layers", 0, "mlp", "limit"), None, "limit"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"), (("layers", 0, "mixer", "right", "groups"), 3, "groups"),
    (("layers", 2, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("layers", 3, "mlp", "kind"), "sparse", "kind")])
def test_a_bad_value_is_refused_by_its_key(path, value, word):
    d = U.config("nip_a")
    at = d
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_no_size_is_refused_in_either_compute_type():
    d = U.config("nip_b")
    d["layers"][1]["mlp"]["ff"] = 100
    d["width"] = 60
    cfg = config_from_dict(d)
    cfg.check_dtype("float32")
    cfg.check_dtype("bfloat16")


def test_the_spec_follows_the_configuration():
    spec = E.config.get_architecture("Nipolorn").build_spec(config_from_dict(U.config("nip_a")))
    assert [l.block for l in spec.layers] == ["sandwich"] * 4 and spec.position.kind == "none" and spec.head == "head"
    assert [None if l.ffn is None else l.ffn.kind for l in spec.layers] == ["gated", "table_experts", None, "table_experts"]
    assert spec.layers[2].norm2 is None and [n for n, _ in spec.layers[2].more_norms] == ["after_mixer"]
    left = dict((n, s) for n, s, _ in spec.layers[0].mixer.params["members"])["left"].params
    assert (left["window"], left["keep_first"], left["head_dim"], left["value_dim"]) == (20, 3, 16, 32)
    model = DecoderModel(spec)
    names = {w.name: w for w in model.weight_specs()}
    assert names["l0.mix.right.in"].shape == (2 * 64 + 2 * 16 + 4, 64) and names["l0.mix.right.conv"].shape == (96, 4)
    assert names["l1.mlp.table"].integer and names["l1.mlp.table"].shape == (300, 2) and "l2.mlp.gate" not in names
    assert names["l3.mlp.e2.down"].shape == (64, 32) and "l3.mlp.shared.gate" not in names and "l1.mlp.shared.up" in names
    cache_need, state_need = model.application_needs()[0]
    assert cache_need == CacheNeed("window", 2, 16, 20, 3, 32)
    assert state_need == {"right.ssm": StateNeed((4, 16, 8)), "right.conv": StateNeed((3, 96))}


def test_random_weights_mode_writes_tables_of_distinct_experts(folders):
    tensors = read_folder(folders["nip_b"])
    table = tensors["l0.mlp.table"]
    assert table.dtype == torch.int32 and tuple(table.shape) == (200, 3)
    assert int(table.min()) >= 0 and int(table.max()) < 4
    assert all(len(set(row)) == 3 for row in table.tolist())
    assert len({tuple(r) for r in table.tolist()}) > 1


# ------------------------------------------------------------------------------ cache
def test_a_window_group_keeps_the_pages_of_the_first_positions():
    need = CacheNeed("window", 1, 16, window=70, keep_first=65, value_dim=24)
    cache = SequenceCache([(need, None)], [None], 1024, None, torch.float32, "cpu")
    g = cache.groups[0]
    assert tuple(g.k[0].shape[1:]) == (1, PAGE, 16) and tuple(g.v[0].shape[1:]) == (1, PAGE, 24) and g.kept_blocks == 2
    s = cache.open()
    cache.reserve([(s, 400)])
    cache.commit([(s, 400)])
    held = [p >= 0 for p in g.held[s]]
    assert held == [True, True, False, False, False, True, True]      # 0..127 kept; the window starts at 331
    for _ in range(200):
        cache.reserve([(s, 1)])
        cache.commit([(s, 1)])
    held = [p >= 0 for p in g.held[s]]
    assert held[:2] == [True, True] and sum(held) == 4 and held[-2:] == [True, True]
    cache.check()
    cache.close(s)
    assert g.pages.free == g.pages.size


def test_state_rows_are_saved_and_put_back():
    cache = SequenceCache([(None, {"a": StateNeed((3,), 0.5), "n": StateNeed((1,), 0, "int32")}), (None, StateNeed((2, 2)))],
                          [None, None], 256, None, torch.float32, "cpu")
    s0, s1 = cache.open(), cache.open()
    cache.states[0]["a"][s1] = 7.0
    cache.states[1][s0] = 3.0
    saved = cache.save_states([s1, -1, s0])
    cache.states[0]["a"].fill_(-1.0)
    cache.states[0]["n"].fill_(9)
    cache.states[1].fill_(-2.0)
    cache.restore_states(saved)
    assert cache.states[0]["a"][s1].tolist() == [7.0] * 3 and cache.states[0]["a"][s0].tolist() == [0.5] * 3
    assert cache.states[0]["n"][s0].item() == 0 and cache.states[1][s0].flatten().tolist() == [3.0] * 4
    assert cache.save_states([-1]) == []


# ------------------------------------------------------------------------------ the plain implementation by itself
def test_plain_window_rule():
    assert P.visible(10, 10, 4, 0) and P.visible(10, 7, 4, 0) and not P.visible(10, 6, 4, 0) and not P.visible(3, 4, 4, 2)
    assert P.visible(10, 1, 4, 2) and not P.visible(10, 2, 4, 2)


def test_plain_recurrence_does_not_depend_on_where_a_sequence_is_cut(plains):
    """The plain convolution and recurrence are whole-sequence functions; cutting the input and carrying
    nothing must differ (the state matters), which is what makes the engine's tests below meaningful."""
    m = plains["nip_a"]
    seq = U.ids(5, 300, 30)
    whole = P.forward(m, seq)
    assert U.row_error(P.forward(m, seq[20:])[-1], whole[-1]) > 1e-3


# ------------------------------------------------------------------------------ the step function over the CPU double
@pytest.mark.parametrize("name", ["nip_a", "nip_b", "nip_c"])
def test_steps_equal_whole_sequences(folders, plains, name):
    """Whole prompts, one token at a time from the first token on, portions down to two tokens, and unequal
    batches decoded together: all give the plain implementation's logits at every position."""
    eng, m = cpu_engine(folders[name]), plains[name]
    vocab = m.cfg["vocab"]
    seqs = [U.ids(10 + i, vocab, n) for i, n in enumerate((150, 1, 40, 97))]
    refs = [P.forward(m, s) for s in seqs]
    got, _ = run_batch(eng, seqs, [len(s) for s in seqs])
    assert max(U.row_error(g, r) for g, r in zip(got, refs)) < 1e-5
    got, _ = run_batch(eng, seqs, [100, 1, 1, 30])                         # prompts, then one token each
    assert max(U.row_error(g, r) for g, r in zip(got, refs)) < 1e-5
    slot, at, rows = eng.open(), 0, []
    for n in (2, 5, 64, 3, 2, 30, 44):                                     # portions of one sequence
        rows.append(eng.step([(slot, seqs[0][at:at + n], list(range(n)))]).numpy())
        at += n
    eng.close(slot)
    assert U.row_error(np.concatenate(rows), refs[0]) < 1e-5
    eng.cache.check()
    assert eng.cache.slots.held == 0 and all(g.pages.held == 0 for g in eng.cache.groups)


def test_slots_and_pages_that_are_used_again_carry_nothing_over(folders, plains):
    eng, m = cpu_engine(folders["nip_a"], max_tokens=256), plains["nip_a"]
    for round_ in range(3):
        seqs = [U.ids(100 * round_ + i, 300, n) for i, n in enumerate((70, 90))]
        got, slots = run_batch(eng, seqs, [60, 2])
        assert sorted(slots) == [0, 1]
        assert max(U.row_error(g, P.forward(m, s)) for g, s in zip(got, seqs)) < 1e-5


def test_greedy_generation_through_the_session(folders, plains):
    for name in ("nip_a", "nip_b"):
        m = plains[name]
        session = E.Session(folders[name], None, max_batch_size=3, dtype="float32", max_tokens=1024, ops=CpuOps(), device="cpu")
        prompts = [U.ids(50 + i, m.cfg["vocab"], n) for i, n in enumerate((5, 23, 1, 9))]
        out = session.generate_batch(prompts, steps=6, temperature=0.0)
        assert out == [P.generate(m, p, 6) for p in prompts]


def test_the_command_line_writes_a_random_model_of_this_design(tmp_path, capsys):
    from ember_cpp_b200 import cli
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(U.config("nip_b")))
    out = tmp_path / "model"
    assert cli.main([str(out), "-", "1", "random-weights", "--config", str(cfg_file), "--seed", "5"]) == 0
    cfg = E.load_config(str(out))
    assert isinstance(cfg, NipolornConfig) and cfg.width == 96
    eng = cpu_engine(str(out), max_tokens=128)
    slot = eng.open()
    logits = eng.step([(slot, U.ids(1, 200, 9), [8])])
    assert tuple(logits.shape) == (1, 200) and bool(torch.isfinite(logits).all())
