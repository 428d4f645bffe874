"""Taredra on the GPU: every mechanism's kernels alone against the plain functions of
tests/plain_taredra.py, then the model through the engine: whole prompts, portions, single
tokens, unequal batches, reused slots, windows' edges, long decoding, greedy generation."""

from types import SimpleNamespace

import pytest
import torch

import plain_taredra as plain
from taredra_helpers import CONFIGS, assert_logits, plain_logits, prompts, spread, write_folder

pytestmark = pytest.mark.gpu

DTYPES = (torch.float32, torch.bfloat16)
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}
PART_TOL = {torch.float32: 2e-5, torch.bfloat16: 5e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("taredra_gpu")
    return {name: write_folder(root / name, name) for name in CONFIGS}


def runtime(dtype):
    from kernel_rush_kawk_b200.csrc import load_kernels
    from kernel_rush_kawk_b200.engine.model import Runtime

    # with the per-head-size attention libraries of the sizes below loaded, bfloat16 steps of many tokens whose key
    # and value heads have one of these sizes take the tensor-core kernel; all others the general one
    return Runtime(torch.device("cuda:0"), dtype, load_kernels((16, 32, 48, 64)))


def rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def context(rt, slots, starts, q_lens, cache):
    from kernel_rush_kawk_b200.engine.step import BatchMeta, StepContext

    meta = BatchMeta(sum(q_lens), len(slots), 0, rt.device)
    meta.fill(slots, starts, [[0] * n for n in q_lens], [])
    return StepContext(rt.ops, meta, cache)


def close(got, ref, dtype, what):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs().max().item()
    tol = PART_TOL[dtype] * ref.abs().max().item()
    assert err <= tol, f"{what}: max |d| = {err:.3e} > {tol:.3e}; first bad row {int(((got - ref).abs() > tol).any(-1).nonzero()[0])}"


def run_part(part, rt, h, pieces, dtype, step_tokens=256, prior=()):
    """One sequence through a mixer part, cut into ``pieces``; ``prior``: sequences that used (and
    gave back) the slot before. No piece is longer than ``step_tokens``, which sizes a window's ring of
    pages (the engine's step function cuts longer steps into passes; here a part is stepped directly)."""
    assert max(pieces) <= step_tokens
    from kernel_rush_kawk_b200.cache import SequenceCache

    cache = SequenceCache([part.cache_need()], 1024, 1, 1024, rt.device, dtype, step_tokens=step_tokens)
    for seq, cuts in list(prior) + [(h, pieces)]:
        slot = cache.alloc()
        got, start = [], 0
        for n in cuts:
            cache.reserve(slot, start + n)
            cache.sync()
            ctx = context(rt, [slot], [start], [n], cache)
            got.append(part.forward(ctx, seq[start:start + n].to(dtype).cuda(), cache.view(0)))
            cache.advance(slot, n)
            start += n
        cache.free(slot)
    rt.ops.check()
    return torch.cat(got)


def as_path(w, dtype):
    """The tensors as the path stores them, and the same values in float64 for the plain functions."""
    stored = {k: v.to(torch.bfloat16) for k, v in w.items()}  # checkpoints hold bfloat16
    return {k: v.to(dtype).cuda() for k, v in stored.items()}, {k: v.double() for k, v in stored.items()}


# ----------------------------------------------------------------------------------------------
# each mechanism alone
# ----------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
def test_scaled_embedding_and_wide_norm(dtype):
    from kernel_rush_kawk_b200.parts import ScaledEmbedding, Stream, WideRMSNorm

    rt = runtime(dtype)
    table = rand((50, 72), 1).to(torch.bfloat16)
    emb = ScaledEmbedding({"vocab": 50, "hidden": 72, "scale": 7.5})
    emb.bind({"table": table.to(dtype).cuda()}, rt)
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32)
    ctx = SimpleNamespace(ops=rt.ops, batch=SimpleNamespace(tokens=ids.cuda(), n_rows=5))
    x = emb.forward(ctx)
    assert x.dtype == torch.float32 and torch.equal(x.cpu(), table.float()[ids.long()] * 7.5)

    gain = (0.2 * rand((72,), 2)).to(torch.bfloat16)
    norm = WideRMSNorm({"size": 72, "eps": 1e-3, "gain_offset": 1.0})
    norm.bind({"weight": gain.to(dtype).cuda()}, rt)
    branch = rand((5, 72), 3, 4.0).to(dtype)
    stream = Stream(x, branch.cuda())
    h = norm.forward(ctx, stream).tensor()
    s = x.double().cpu() + branch.double()
    assert stream.branch is None and stream.x.dtype == torch.float32
    assert torch.equal(stream.x.cpu(), (x.cpu() + branch.float()))  # the sum is 32-bit, not rounded to the path's dtype
    assert h.dtype == dtype
    close(h, plain.centered_norm(s, gain.double(), 1e-3), dtype, "norm with a pending branch")
    alone = norm.forward(ctx, Stream(x)).tensor()
    close(alone, plain.centered_norm(x.double().cpu(), gain.double(), 1e-3), dtype, "norm alone")
    plain_gain = WideRMSNorm({"size": 72, "eps": 1e-3})  # offset 0: the weight is the gain itself
    plain_gain.bind({"weight": (1 + gain.float()).to(dtype).cuda()}, rt)
    close(plain_gain.forward(ctx, Stream(x)).tensor(),
          plain.unit_rms(x.double().cpu(), 1e-3) * (1 + gain.float()).to(dtype).double(), dtype, "norm, offset 0")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [3, 40])
def test_gated_mlp(dtype, rows):
    from kernel_rush_kawk_b200.parts import GatedMLP

    rt = runtime(dtype)
    w = {"gate": rand((88, 64), 1, 0.3), "up": rand((88, 64), 2, 0.3), "down": rand((64, 88), 3, 0.3)}
    dev, ref = as_path(w, dtype)
    part = GatedMLP({"hidden": 64, "intermediate": 88, "activation": "gelu_tanh"})
    part.bind(dev, rt)
    h = rand((rows, 64), 4, 2.0).to(dtype)
    got = part.forward(SimpleNamespace(ops=rt.ops), h.cuda())
    close(got, plain.gated_ff(h.double(), ref["gate"], ref["up"], ref["down"]), dtype, "gated feed-forward")


ATTN_SHAPES = [  # hidden, heads, kv_heads, dim, vdim, window, rot, base
    (72, 6, 3, 16, 16, 20, 16, 1e4),
    (64, 4, 1, 32, 64, 70, 8, 2e4),
    (40, 2, 2, 24, 8, 7, 24, 50.0),
    (48, 3, 1, 8, 40, 130, 2, 10.0),
    (64, 2, 1, 64, 64, 1, 64, 1e4),
    (96, 4, 2, 48, 48, 40, 32, 1e4),
    (40, 10, 1, 8, 8, 90, 4, 30.0),
]


def attention_part(shape, dtype, rt, seed=0):
    from kernel_rush_kawk_b200.parts import SinkWindowAttention

    C, H, G, D, Dv, window, rot, base = shape
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.4, "mask": {"size": window},
         "rot": {"dims": rot, "base": base}}
    part = SinkWindowAttention({"hidden": C, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.4, "window": window,
                                "rot_dims": rot, "rot_base": base, "value_norm": True, "sink": True, "eps": 1e-5})
    w = {"q": rand((H * D, C), seed + 1, 0.4), "k": rand((G * D, C), seed + 2, 0.4), "v": rand((G * Dv, C), seed + 3, 0.3),
         "o": rand((C, H * Dv), seed + 4, 0.2), "sink": rand((H,), seed + 5, 2.0)}
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    return part, m, ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTN_SHAPES)
def test_sink_window_attention_alone(dtype, shape):
    rt = runtime(dtype)
    part, m, ref = attention_part(shape, dtype, rt)
    T = 150
    h = rand((T, shape[0]), 9).to(dtype)
    want = plain.windowed_branch(h.double(), ref, "", m, 1e-5, torch.arange(T))
    for pieces in ([T], [63, 2, 64, 21], [100] + [1] * 50):
        got = run_part(part, rt, h, pieces, dtype)
        close(got, want, dtype, f"attention {shape}, pieces {pieces[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_counts_once_and_has_no_value(dtype):
    """One head's sink far above every score: that head's output vanishes; far below: an ordinary softmax."""  # noqa
    rt = runtime(dtype)
    shape = (32, 2, 1, 16, 16, 12, 16, 1e4)
    part, m, ref = attention_part(shape, dtype, rt)
    part.sink = torch.tensor([80.0, -80.0], device="cuda")
    ref["sink"] = torch.tensor([80.0, -80.0], dtype=torch.float64)
    part._w_out = torch.eye(32, dtype=dtype, device="cuda")  # look at the heads themselves
    ref["o"] = torch.eye(32, dtype=torch.float64)
    h = rand((40, 32), 3).to(dtype)
    got = run_part(part, rt, h, [40], dtype).double().cpu()
    want = plain.windowed_branch(h.double(), ref, "", m, 1e-5, torch.arange(40))
    close(got, want, dtype, "sinks of +80 and -80")
    assert got[:, :16].abs().max() < 1e-6 and got[:, 16:].abs().max() > 0.1


def spike_case(window, T, spike_at, dtype):
    """Queries, keys and values given directly: every query points along e0, the key at ``spike_at``
    too (score 40 above the others), its value is (100, 100, ...). The outputs show at which
    positions that one key is seen."""
    D = 16
    q = rand((T, 1, D), 1, 0.05); q[:, 0, 0] = 8.0
    k = rand((T, 1, D), 2, 0.05); k[spike_at, 0, 0] = 5.0
    v = rand((T, 1, D), 3, 1.0); v[spike_at] = 100.0
    return q.to(dtype), k.to(dtype), v.to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, spike_at, T", [(10, 3, 40), (64, 0, 140), (65, 63, 200), (300, 5, 420), (73, 55, 150)])
def test_one_key_at_the_windows_edge(dtype, window, spike_at, T):
    """The kernels alone on crafted heads, whole and with the edge crossed token by token: the key is
    seen up to position spike + window - 1 and not from spike + window on (also where the edge
    lies on a page border, and for a key hundreds of tokens back)."""
    from kernel_rush_kawk_b200.cache import SequenceCache
    from kernel_rush_kawk_b200.parts import KVNeed

    rt = runtime(dtype)
    q, k, v = spike_case(window, T, spike_at, dtype)
    sink = torch.zeros(1, dtype=torch.float64)
    want = plain.sink_window_attention(q.double(), k.double(), v.double(), 1.0, window, sink)[:, 0]
    edge = spike_at + window
    assert want[edge - 1, 0] > 90 and (edge >= T or want[edge, 0] < 10)
    no_freq = torch.zeros(0, device="cuda")
    for pieces in ([T], [min(edge - 2, T - 1)] + [1] * (T - min(edge - 2, T - 1)), [2] * (T // 2)):
        cache = SequenceCache([KVNeed(1, 16, window)], 1024, 1, 1024, rt.device, dtype, step_tokens=T)
        slot = cache.alloc()
        outs, start = [], 0
        for n in pieces:
            cache.reserve(slot, start + n)
            cache.sync()
            ctx = context(rt, [slot], [start], [n], cache)
            proj = torch.cat([q[start:start + n, 0], k[start:start + n, 0], v[start:start + n, 0]], dim=1).cuda().contiguous()
            out = torch.empty((n, 16), dtype=dtype, device="cuda")
            rt.ops.rotate_norm_write(proj, 0, 16, 32, 1, 1, 16, 16, no_freq, 0, None, ctx.batch, cache.view(0))
            rt.ops.sink_attention(proj, 0, 1, 16, 16, sink.float().cuda(), 1.0, window, ctx.batch, cache.view(0), out, 0, 1.0)
            outs.append(out)
            cache.advance(slot, n)
            start += n
        close(torch.cat(outs), want, dtype, f"window {window}, key at {spike_at}, pieces {pieces[:3]}")


STATE_SHAPES = [(64, 3, 16, 8), (48, 1, 48, 16), (96, 2, 32, 5), (64, 1, 64, 16), (40, 5, 8, 3), (64, 1, 128, 4),
                (40, 2, 20, 3), (30, 2, 5, 2), (72, 1, 100, 40), (48, 1, 160, 6), (32, 1, 256, 4)]


def state_weights(kind, C, H, N, R, seed):
    HN = H * N
    w = {k: rand((HN, C), seed + i, 0.25) for i, k in enumerate(("r", "k", "v", "g"))}
    w.update({"w1": rand((R, C), seed + 5, 0.3), "w2": rand((HN, R), seed + 6, 0.8), "w0": rand((HN,), seed + 7, 1.0),
              "norm": 1 + rand((HN,), seed + 8, 0.2), "o": rand((C, HN), seed + 9, 0.2)})
    if kind == "delta":
        w.update({"a": rand((HN, C), seed + 10, 0.3), "a.b": rand((HN,), seed + 11, 1.0)})
    else:
        w.update({"u": rand((H, N), seed + 12, 0.5)})
        w.update({"mu." + s: rand((C,), seed + 13 + i, 0.4) + 0.5 for i, s in enumerate("rkvgw")})
    return w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", STATE_SHAPES)
@pytest.mark.parametrize("kind", ["delta", "wkv"])
def test_recurrent_mixers_alone(dtype, shape, kind):
    """Whole, in pieces down to two tokens, token by token, and in a slot that another sequence used
    before (the state must start from zero again)."""
    from kernel_rush_kawk_b200.parts import DeltaRule, TimeMixWKV

    rt = runtime(dtype)
    C, H, N, R = shape
    cls = DeltaRule if kind == "delta" else TimeMixWKV
    part = cls({"hidden": C, "heads": H, "dim": N, "rank": R, "eps": 1e-5})
    w = state_weights(kind, C, H, N, R, 20)
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    T = 70
    h = rand((T, C), 5).to(dtype)
    m = {"heads": H, "dim": N}
    want = (plain.delta_branch if kind == "delta" else plain.wkv_mixer)(h.double(), ref, "", m, 1e-5)
    other = rand((9, C), 6).to(dtype)
    for pieces, prior in (([T], ()), ([17, 2, 33, 16, 2], ()), ([30] + [1] * 40, ()), ([T], [(other, [9])])):
        got = run_part(part, rt, h, pieces, dtype, prior=prior)
        close(got, want, dtype, f"{kind} {shape}, pieces {pieces[:4]}, prior {len(prior)}")


def test_scans_do_not_depend_on_the_cut_to_the_bit():
    """32-bit: the state after a sequence and every output are bit-equal whole and in pieces."""
    from kernel_rush_kawk_b200.parts import DeltaRule

    rt = runtime(torch.float32)
    part = DeltaRule({"hidden": 48, "heads": 2, "dim": 24, "rank": 6, "eps": 1e-6})
    dev, _ = as_path(state_weights("delta", 48, 2, 24, 6, 40), torch.float32)
    part.bind(dev, rt)
    h = rand((90, 48), 8).float()
    whole = run_part(part, rt, h, [90], torch.float32)
    for pieces in ([1] * 90, [16, 16, 1, 15, 42], [89, 1]):
        assert torch.equal(run_part(part, rt, h, pieces, torch.float32), whole), pieces
    # the optional three-kernel form of many-token steps forms the same sums in the same order
    rt.ops.split_recurrence = True
    try:
        for pieces in ([90], [40, 33, 17]):
            assert torch.equal(run_part(part, rt, h, pieces, torch.float32), whole), ("split", pieces)
    finally:
        rt.ops.split_recurrence = False


@pytest.mark.parametrize("dtype", DTYPES)
def test_parallel_mixer_alone(dtype):
    """Two branches on one input: one stacked input product, one output product over both branches' columns."""
    from kernel_rush_kawk_b200.parts import ParallelMixer

    rt = runtime(dtype)
    C = 56
    left = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "mask": {"size": 11}, "rot": {"dims": 8, "base": 300.0}}
    right = {"heads": 3, "dim": 16}
    m = {"left": left, "right": right, "left_scale": 0.6, "right_scale": 1.7}
    part = ParallelMixer({"hidden": C, "branches": [
        {"name": "left", "kind": "sink_window_attention", "scale": 0.6,
         "params": {"hidden": C, "heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "window": 11, "rot_dims": 8,
                    "rot_base": 300.0, "value_norm": True, "sink": True, "eps": 1e-5}},
        {"name": "right", "kind": "delta_rule", "scale": 1.7,
         "params": {"hidden": C, "heads": 3, "dim": 16, "rank": 7, "eps": 1e-5}}]})
    w = {"left.q": rand((64, C), 1, 0.4), "left.k": rand((32, C), 2, 0.4), "left.v": rand((48, C), 3, 0.3),
         "left.o": rand((C, 96), 4, 0.2), "left.sink": rand((4,), 5, 1.0)}
    w.update({"right." + k: v for k, v in state_weights("delta", C, 3, 16, 7, 60).items()})
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    T = 50
    h = rand((T, C), 7).to(dtype)
    want = plain.parallel_mixer(h.double(), ref, "", m, 1e-5, torch.arange(T))
    for pieces in ([T], [20, 2, 28], [1] * T):
        close(run_part(part, rt, h, pieces, dtype), want, dtype, f"parallel mixer, pieces {pieces[:3]}")


# ----------------------------------------------------------------------------------------------
# the model through the engine
# ----------------------------------------------------------------------------------------------

def engine_for(folder, dtype, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype=dtype, max_tokens=4096, max_slots=6, max_context=1024, step_tokens=64)
    args.update(kw)
    return Engine(folder, **args)


def feed(engine, slot, seq, pieces):
    from kernel_rush_kawk_b200 import StepEntry

    outs, start = [], 0
    for n in pieces:
        outs.append(engine.step([StepEntry(slot, seq[start:start + n], list(range(n)))]).clone())
        start += n
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_portions_and_single_tokens(folders, name, dtype):
    engine = engine_for(folders[name], dtype)
    seq = prompts(name, [200], seed=11)[0]
    ref = plain_logits(folders[name], seq)
    for pieces in ([200], [2] * 100, [64, 64, 72], [3, 61, 1, 63, 70, 2], [150] + [1] * 50, [1] * 200):
        slot = engine.cache.alloc()
        assert_logits(feed(engine, slot, seq, pieces), ref, dtype, f"{name} pieces {pieces[:4]}")
        engine.cache.free(slot)
    engine.cache.check()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_first_tokens_of_a_sequence(folders, name):
    """Positions 0, 1, 2: no previous token for the token shift, an empty state, a window that holds
    fewer keys than its size, the sink beside a single key."""
    engine = engine_for(folders[name], "float32")
    for n in (1, 2, 3):
        seq = prompts(name, [n], seed=12 + n)[0]
        slot = engine.cache.alloc()
        assert_logits(feed(engine, slot, seq, [n]), plain_logits(folders[name], seq), "float32", f"{name}, {n} tokens")
        engine.cache.free(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_equal_each_alone(folders, dtype):
    from kernel_rush_kawk_b200 import StepEntry

    name = "tb"
    engine = engine_for(folders[name], dtype)
    seqs = prompts(name, [1, 130, 47, 260], seed=13)
    cut = [1, 100, 30, 200]
    alone = []
    for seq, c in zip(seqs, cut):
        slot = engine.cache.alloc()
        alone.append(feed(engine, slot, seq, [c] + [1] * (len(seq) - c)))
        engine.cache.free(slot)
    slots = [engine.cache.alloc() for _ in seqs]
    got = [[] for _ in seqs]
    out = engine.step([StepEntry(sl, s[:c], list(range(c))) for sl, s, c in zip(slots, seqs, cut)])
    r = 0
    for i, c in enumerate(cut):
        got[i].append(out[r:r + c].clone()); r += c
    fed = list(cut)
    while any(f < len(s) for f, s in zip(fed, seqs)):
        live = [i for i in range(len(seqs)) if fed[i] < len(seqs[i])]
        out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1].clone()); fed[i] += 1
    for i, seq in enumerate(seqs):
        both = torch.cat(got[i])
        assert_logits(both, plain_logits(folders[name], seq), dtype, f"request {i} in the batch")
        if dtype == "float32" and len(seq) > 1:
            # every sum of the 32-bit path is ordered per row, so nothing depends on the batch. (A prompt of one
            # token is a single-token step alone and a row of a many-token step in the batch: two kernels for the
            # attention, equal up to rounding.)
            assert torch.equal(both, alone[i]), f"request {i}: batched and alone differ"
        else:
            assert spread(both, alone[i]).max() < 2e-2


def test_slots_and_pages_that_are_freed_and_used_again(folders):
    """Two slots, five requests one after another through them, pages handed around: every request's
    logits are those of the request alone in a fresh engine's terms (the plain implementation)."""
    from kernel_rush_kawk_b200 import StepEntry

    name = "ta"
    engine = engine_for(folders[name], "float32", max_tokens=512, max_slots=2)
    seqs = prompts(name, [100, 190, 64, 129, 30], seed=14)
    waiting = list(range(len(seqs)))
    live = {}
    while waiting or live:
        while waiting and engine.cache.live < 2:
            i = waiting.pop(0)
            live[i] = [engine.cache.alloc(), 0, []]
            half = len(seqs[i]) // 2
            live[i][2].append(engine.step([StepEntry(live[i][0], seqs[i][:half], list(range(half)))]).clone())
            live[i][1] = half
        ids = sorted(live)
        out = engine.step([StepEntry(live[i][0], [seqs[i][live[i][1]]], [0]) for i in ids])
        for r, i in enumerate(ids):
            live[i][2].append(out[r:r + 1].clone())
            live[i][1] += 1
            if live[i][1] == len(seqs[i]):
                assert_logits(torch.cat(live[i][2]), plain_logits(folders[name], seqs[i]), "float32", f"request {i}")
                engine.cache.free(live.pop(i)[0])
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_every_window_and_ring(folders, dtype):
    """Six hundred single-token steps after a short prompt: windows of 5 to 70 keys pass over decoded
    tokens many times and the windows' rings of pages are reused; the state carries all of it."""
    name = "tb"
    engine = engine_for(folders[name], dtype, step_tokens=16)
    seq = prompts(name, [620], seed=15)[0]
    slot = engine.cache.alloc()
    got = feed(engine, slot, seq, [20] + [1] * 600)
    assert_logits(got, plain_logits(folders[name], seq), dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_single_token_steps_with_the_fused_attention_option(folders, dtype):
    """The option that rotates, normalises and writes the new key and value inside the single-token attention
    kernel: the same logits as the plain implementation, through captured steps of an unequal batch."""
    from kernel_rush_kawk_b200 import StepEntry

    name = "tb"
    engine = engine_for(folders[name], dtype)
    engine.ops.fuse_single_token_attention = True
    try:
        seqs = prompts(name, [90, 150], seed=18)
        slots = [engine.cache.alloc() for _ in seqs]
        cut = [10, 75]
        got = [[engine.step([StepEntry(sl, s[:c], list(range(c)))]).clone()] for sl, s, c in zip(slots, seqs, cut)]
        fed = list(cut)
        while any(f < len(s) for f, s in zip(fed, seqs)):
            live = [i for i in range(2) if fed[i] < len(seqs[i])]
            out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1].clone()); fed[i] += 1
        for i, seq in enumerate(seqs):
            assert_logits(torch.cat(got[i]), plain_logits(folders[name], seq), dtype, f"fused option, request {i}")
    finally:
        engine.ops.fuse_single_token_attention = False


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """Engine.generate (the scheduler, the captured single-token step, the selection kernel) against
    the plain implementation's argmax, token by token, ties within the arithmetic's noise allowed."""
    name = "ta"
    engine = engine_for(folders[name], dtype, max_tokens=None)
    seqs = prompts(name, [5, 33, 1, 70], seed=16)
    steps = list(engine.generate(seqs, 12))
    assert len(steps) == 12 and engine.stepper.use_graphs
    cfg, w = plain.read_folder(folders[name], torch.float64)
    for i, seq in enumerate(seqs):
        seq = list(seq)
        for t in range(12):
            ref = plain.forward(cfg, w, seq)[-1]
            tok = steps[t][i]
            allowed = (1e-4 if dtype == "float32" else 5e-2) * (ref - ref.mean()).pow(2).mean().sqrt().item()
            assert ref.max().item() - ref[tok].item() <= allowed, f"request {i} step {t}: token {tok} is not the plain choice"
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(folders, dtype, tmp_path):
    """bin/trace_run on a model folder of this design: requests alone, decoded, and unequal requests in one batch
    that shrinks as they end, with --max-tokens counting tokens only (no rounding to pages)."""
    from test_replay_gpu import Trace, run_trace

    name = "ta"
    vocab = CONFIGS[name]["vocab"]
    seqs = prompts(name, [1, 97, 130, 45], seed=17)
    trace = Trace()
    for i, toks in enumerate(seqs):
        trace.batch({f"r{i}w": toks}, [len(toks)])
    trace.batch({"r1d": seqs[1]}, [len(seqs[1]) - 40])
    trace.batch({"r0b": seqs[0], "r1b": seqs[1], "r2b": seqs[2], "r3b": seqs[3]}, [1, 65, 98, 13])
    got = run_trace(folders[name], dtype, trace, tmp_path / "out", sum(len(s) for s in seqs), vocab)
    assert len(got) >= sum(len(s) for s in seqs)
    for (rid, pos), rows in got.items():
        ref = plain_logits(folders[name], seqs[int(rid[1])])[pos:pos + 1]
        for row in rows:
            assert_logits(row[None], ref, dtype, f"{dtype} request {rid} position {pos}")
