"""Disorax without a GPU: its configuration, its plan, the cache's storage for it, and the engine's step
logic over it with the kernels replaced by their plain torch restatement (tests/torch_ops.py), against
the plain implementation (tests/plain_disorax.py)."""

import copy

import pytest
import torch

from disorax_helpers import CONFIGS, assert_logits, config, plain_logits, prompts, write_folder
from torch_ops import TorchOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("disorax")
    return {name: write_folder(root / name, name) for name in CONFIGS}


def cpu_engine(folder, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype="float32", device="cpu", ops=TorchOps(torch.float32), max_tokens=1024, max_slots=5,
                max_context=512, use_cuda_graphs=False)
    args.update(kw)
    return Engine(folder, **args)


def test_config_reads_back_and_is_found_by_its_name(folders):
    from kernel_rush_kawk_b200 import DisoraxConfig, read_config

    for name in CONFIGS:
        arch, cfg = read_config(folders[name])
        assert arch.name == "Disorax" and isinstance(cfg, DisoraxConfig)
        assert DisoraxConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.residual_mult == CONFIGS[name]["residual_mult"]


@pytest.mark.parametrize("damage, word", [
    (lambda c: c["layers"][1].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][3]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 8), "blend"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0].__setitem__("mlp", {"kind": "dense", "ff": 8}), "moe"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_config_faults_are_named(damage, word):
    from kernel_rush_kawk_b200 import ConfigError, DisoraxConfig

    raw = copy.deepcopy(CONFIGS["da"])
    damage(raw)
    with pytest.raises(ConfigError, match=word):
        DisoraxConfig.from_dict(raw)


def test_plan_names_every_tensor_and_each_layer_asks_the_cache_for_what_it_keeps():
    from kernel_rush_kawk_b200.config.registry import get_architecture
    from kernel_rush_kawk_b200.engine.model import PartTree
    from kernel_rush_kawk_b200.parts import KVNeed

    cfg = config("da")
    tree = PartTree(get_architecture("Disorax").plan(cfg))
    names = tree.expected_tensors()
    assert tuple(names["l0.mix.g"].shape) == (4 * 24, 64) and tuple(names["l1.mix.g"].shape) == (3, 64)
    assert tuple(names["l0.mix.vmix"].shape) == () and "l1.mix.vmix" not in names
    assert tuple(names["l3.mix.sink"].shape) == (2,) and "l1.mix.sink" not in names
    assert "l2.mlp.shared.gate" not in names and tuple(names["l0.mlp.shared.sg"].shape) == (1, 64)
    assert "l1.norm2" not in names and "head" in names and "final.norm" in names
    needs = tree.cache_needs()
    assert needs[0] == KVNeed(2, 16, 10, 24, keep_first=3)
    assert needs[1] == KVNeed(1, 24, None, values=False)  # a latent row serves as key and as value
    assert needs[3] == KVNeed(1, 16, 6, values=False)


def test_kept_first_pages_stay_out_of_the_ring():
    """A window group with kept first tokens: the first pages are held for good, later ones go round."""
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import KVNeed

    cache = SequenceCache([KVNeed(1, 8, 20, keep_first=70), KVNeed(1, 8, None, values=False)], 64 * 40, 2, 64 * 40, "cpu",
                          torch.float32, step_tokens=44)
    kv, latent = cache.view(0), cache.view(1)
    assert kv.keep_pages == 2 and kv.width == 2 + 2  # ceil(70 / 64) kept, ceil((20 + 44 - 1) / 64) + 1 in the ring
    assert latent.v.data_ptr() == latent.k.data_ptr() and latent.keep_pages == 0
    slot = cache.alloc()
    cache.reserve(slot, 64 * 30)
    cache.sync()
    ops = TorchOps(torch.float32)
    from torch_ops import _entry
    entries = _entry(kv, torch.arange(0, 64 * 30, 64))
    assert entries[:2].tolist() == [0, 1] and set(entries[2:].tolist()) == {2, 3}
    assert entries[2:6].tolist() == [2, 3, 2, 3]
    cache.free(slot)
    cache.check()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_portions_and_single_tokens_agree_with_the_plain_implementation(folders, name):
    from kernel_rush_kawk_b200 import StepEntry

    eng = cpu_engine(folders[name], step_tokens=24)  # steps longer than 24 tokens are cut into passes: the rings turn
    ids = prompts(name, [130])[0]
    ref = plain_logits(folders[name], ids)
    for pieces in ([130], [70, 2, 3, 55], [100] + [1] * 30):
        slot = eng.cache.alloc()
        got, start = [], 0
        for n in pieces:
            got.append(eng.step([StepEntry(slot, ids[start:start + n], list(range(n)))]))
            start += n
        eng.cache.free(slot)
        assert_logits(torch.cat(got), ref, "float32", f"{name}, pieces {pieces[:4]}")
    eng.cache.check()


def test_unequal_batch_against_each_alone(folders):
    from kernel_rush_kawk_b200 import StepEntry

    eng = cpu_engine(folders["da"])
    seqs = prompts("da", [40, 1, 75, 13], seed=3)
    slots = [eng.cache.alloc() for _ in seqs]
    first = eng.step([StepEntry(s, ids[:-2] if len(ids) > 2 else ids, [len(ids[:-2] if len(ids) > 2 else ids) - 1])
                      for s, ids in zip(slots, seqs)])
    for i, ids in enumerate(seqs):
        ref = plain_logits(folders["da"], ids)
        n = len(ids) - 2 if len(ids) > 2 else len(ids)
        assert_logits(first[i:i + 1], ref[n - 1:n], "float32", f"batched prompt {i}")
    live = [(s, ids) for s, ids in zip(slots, seqs) if len(ids) > 2]
    for back in (2, 1):
        got = eng.step([StepEntry(s, [ids[-back]], [0]) for s, ids in live])
        for i, (s, ids) in enumerate(live):
            ref = plain_logits(folders["da"], ids)
            assert_logits(got[i:i + 1], ref[len(ids) - back:len(ids) - back + 1], "float32", f"batched token of sequence {i}")
