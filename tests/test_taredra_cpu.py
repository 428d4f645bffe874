"""Taredra without a GPU: its configuration, its plan, the cache's storage for it, and the engine's
step and generation logic over it with the kernels replaced by their plain torch restatement
(tests/torch_ops.py), against the plain implementation (tests/plain_taredra.py)."""

import copy
import json

import pytest
import torch

import plain_taredra as plain
from taredra_helpers import CONFIGS, assert_logits, config, plain_logits, prompts, write_folder
from torch_ops import TorchOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("taredra")
    return {name: write_folder(root / name, name) for name in CONFIGS}


def cpu_engine(folder, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype="float32", device="cpu", ops=TorchOps(torch.float32), max_tokens=1024, max_slots=5,
                max_context=512, use_cuda_graphs=False)
    args.update(kw)
    return Engine(folder, **args)


def test_config_reads_back_and_names_its_architecture_with_one_string(folders):
    from kernel_rush_kawk_b200 import TaredraConfig, read_config

    for name in CONFIGS:
        arch, cfg = read_config(folders[name])
        assert arch.name == "Taredra" and isinstance(cfg, TaredraConfig)
        assert TaredraConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.layers[0]["type"] == CONFIGS[name]["layers"][0]["type"]


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][1].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0].__setitem__("mlp", {"kind": "routed", "ff": 8}), "dense"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_config_faults_are_named(damage, word):
    from kernel_rush_kawk_b200 import ConfigError, TaredraConfig

    raw = copy.deepcopy(CONFIGS["ta"])
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        TaredraConfig.from_dict(raw)


def test_the_rank_of_a_decay_comes_from_the_checkpoint(folders, tmp_path):
    """The configuration file need not give it: the engine reads it off the tensors' shapes."""
    from kernel_rush_kawk_b200 import Engine

    raw = json.loads((folders["ta"] / "config.json").read_text())
    for layer in raw["layers"]:
        layer["mixer"].pop("rank", None)
        layer["mixer"].get("right", {}).pop("rank", None)
    (tmp_path / "config.json").write_text(json.dumps(raw))
    (tmp_path / "model.safetensors").write_bytes((folders["ta"] / "model.safetensors").read_bytes())
    engine = Engine(tmp_path, dtype="float32", device="cpu", ops=TorchOps(torch.float32), max_tokens=128, max_slots=1)
    assert engine.config.layers[0]["mixer"]["rank"] == 8 and engine.config.layers[2]["mixer"]["right"]["rank"] == 12


def test_plan_names_every_tensor_of_the_checkpoint(folders):
    from safetensors import safe_open
    from kernel_rush_kawk_b200.engine.model import expected_tensors
    from kernel_rush_kawk_b200.models.taredra import taredra_plan

    for name in CONFIGS:
        plan = taredra_plan(config(name))
        with safe_open(str(folders[name] / "model.safetensors"), framework="pt") as f:
            stored = {k: tuple(f.get_slice(k).get_shape()) for k in f.keys()}
        assert {k: tuple(v.shape) for k, v in expected_tensors(plan).items()} == stored
        assert plan.layers[0].feed_forward is not None or plan.layers[1].feed_forward is not None
        assert any(layer.feed_forward is None for layer in plan.layers)


def test_a_missing_or_misshapen_tensor_is_reported(folders, tmp_path):
    from safetensors.torch import load_file, save_file
    from kernel_rush_kawk_b200 import WeightError

    tensors = load_file(str(folders["ta"] / "model.safetensors"))
    tensors.pop("l1.mix.left.sink")
    tensors["l0.mix.u"] = tensors["l0.mix.u"][:, :8].contiguous()
    save_file(tensors, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text((folders["ta"] / "config.json").read_text())
    with pytest.raises(WeightError) as err:
        cpu_engine(tmp_path)
    assert "l1.mix.left.sink" in err.value.missing and "l0.mix.u" in err.value.wrong_shape


def test_cache_storage_of_a_run_with_several_needs():
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import KVNeed, StateNeed

    needs = [(KVNeed(2, 16, 10, 32), StateNeed((3, 16, 16))), (StateNeed((2, 8, 8)), StateNeed((40,))),
             (KVNeed(2, 16, 10, 32), StateNeed((3, 16, 16))), StateNeed((40,)), None]
    cache = SequenceCache(needs, 512, 3, 256, "cpu", torch.float32, step_tokens=20)
    kv, st = cache.view(0)
    assert kv.k.shape[1:] == (2, 64, 16) and kv.v.shape[1:] == (2, 64, 32) and kv.v_dim == 32 and kv.window == 10
    assert st.state.shape == (3, 3, 16, 16)
    kv2, st2 = cache.view(2)
    assert kv2.k.data_ptr() != kv.k.data_ptr() and st2.state.data_ptr() != st.state.data_ptr()
    a, b = cache.view(1)
    assert a.state.shape == (3, 2, 8, 8) and b.state.shape == (3, 40)
    assert cache.view(3).state.shape == (3, 40) and cache.view(3).state.data_ptr() != b.state.data_ptr()
    assert cache.view(4) is None
    slot = cache.alloc()
    st.state[slot] += 1.0
    b.state[slot] += 2.0
    cache.free(slot)
    again = cache.alloc()
    assert again == slot and float(st.state[slot].abs().sum()) == 0.0 and float(b.state[slot].abs().sum()) == 0.0
    cache.free(again)
    cache.check()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_pieces_and_single_tokens_agree_with_plain(folders, name):
    from kernel_rush_kawk_b200 import StepEntry

    engine = cpu_engine(folders[name], step_tokens=24)  # windows' rings shorter than the sequences
    seqs = prompts(name, [90, 5, 41], seed=3)
    refs = [plain_logits(folders[name], s) for s in seqs]
    slots = [engine.cache.alloc() for _ in seqs]
    cuts = [(37, 80), (1, 3), (2, 40)]
    got = [[] for _ in seqs]
    fed = [0] * len(seqs)
    for k in range(2):
        entries = [StepEntry(sl, s[fed[i]:c[k]], list(range(c[k] - fed[i]))) for i, (sl, s, c) in enumerate(zip(slots, seqs, cuts))]
        out = engine.step(entries)
        r = 0
        for i, c in enumerate(cuts):
            got[i].append(out[r:r + c[k] - fed[i]]); r += c[k] - fed[i]; fed[i] = c[k]
    while any(f < len(s) for f, s in zip(fed, seqs)):
        live = [i for i in range(len(seqs)) if fed[i] < len(seqs[i])]
        out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1]); fed[i] += 1
    for i, ref in enumerate(refs):
        assert_logits(torch.cat(got[i]), ref, "float32", f"{name} request {i}")
    for s in slots:
        engine.cache.free(s)
    engine.cache.check()


def test_a_freed_slot_starts_from_an_empty_state(folders):
    from kernel_rush_kawk_b200 import StepEntry

    name = "tb"
    engine = cpu_engine(folders[name], max_slots=1)
    a, b = prompts(name, [50, 23], seed=4)
    for seq in (a, b, a):
        slot = engine.cache.alloc()
        out = engine.step([StepEntry(slot, seq, [len(seq) - 1])])
        assert_logits(out, plain_logits(folders[name], seq)[-1:], "float32", "reused slot")
        engine.cache.free(slot)


def test_greedy_generation_through_the_engine(folders):
    name = "ta"
    engine = cpu_engine(folders[name])
    seqs = prompts(name, [6, 19, 2], seed=5)
    steps = list(engine.generate(seqs, 5))
    assert len(steps) == 5
    cfg, w = plain.read_folder(folders[name], torch.float64)
    for i, seq in enumerate(seqs):
        seq = list(seq)
        for t in range(5):
            ref = plain.forward(cfg, w, seq)[-1]
            tok = steps[t][i]
            assert ref.max().item() - ref[tok].item() <= 1e-4 * ref.abs().max().item(), f"request {i} step {t}"
            seq.append(tok)
