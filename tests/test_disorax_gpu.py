"""Disorax on the GPU: every mechanism's kernels alone against the plain functions of
tests/plain_disorax.py, then the model through the engine: whole prompts, portions, single tokens,
unequal batches, reused slots, windows' and kept tokens' edges, rings that turn, long decoding,
greedy generation and trace replay."""

import io
import json
from types import SimpleNamespace

import pytest
import torch

import plain_disorax as plain
from disorax_helpers import CONFIGS, assert_logits, plain_logits, prompts, spread, write_folder

pytestmark = pytest.mark.gpu

DTYPES = (torch.float32, torch.bfloat16)
NAME = {torch.float32: "float32", torch.bfloat16: "bfloat16"}
PART_TOL = {torch.float32: 3e-5, torch.bfloat16: 5e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("disorax_gpu")
    return {name: write_folder(root / name, name) for name in CONFIGS}


def runtime(dtype):
    from kernel_rush_kawk_b200.csrc import load_kernels
    from kernel_rush_kawk_b200.engine.model import Runtime

    # with the per-head-size attention libraries of these sizes loaded, bfloat16 steps of many tokens whose key and
    # value heads have one of them take the tensor-core kernel; all others the general one
    return Runtime(torch.device("cuda:0"), dtype, load_kernels((16, 32)))


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


def run_part(part, rt, h, pieces, dtype, step_tokens=256, prior=(), before=None):
    """One sequence through a mixer part, cut into ``pieces``; ``prior``: sequences that used (and gave
    back) the slot before; ``before(ctx, start, n)`` prepares what an earlier layer would have left."""
    assert max(pieces) <= step_tokens
    from kernel_rush_kawk_b200.cache import SequenceCache

    cache = SequenceCache([part.cache_need()], 2048, 1, 2048, rt.device, dtype, step_tokens=step_tokens)
    for seq, cuts in list(prior) + [(h, pieces)]:
        slot = cache.alloc()
        got, start = [], 0
        for n in cuts:
            cache.reserve(slot, start + n)
            cache.sync()
            ctx = context(rt, [slot], [start], [n], cache)
            if before is not None and seq is h:
                before(ctx, start, n)
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
@pytest.mark.parametrize("width", [72, 50])
def test_two_norms_of_one_x_with_two_pending_outputs_and_a_multiplier(dtype, width):
    from kernel_rush_kawk_b200.parts import Stream, WideRMSNorm

    rt = runtime(dtype)
    ctx = SimpleNamespace(ops=rt.ops)
    x = rand((7, width), 1, 3.0).cuda()
    a, b = rand((7, width), 2, 2.0).to(dtype), rand((7, width), 3, 2.0).to(dtype)
    g1, g2 = (1 + 0.3 * rand((width,), 4)).to(torch.bfloat16), (1 + 0.3 * rand((width,), 5)).to(torch.bfloat16)
    n1, n2 = WideRMSNorm({"size": width, "eps": 1e-4}), WideRMSNorm({"size": width, "eps": 1e-4})
    n1.bind({"weight": g1.to(dtype).cuda()}, rt)
    n2.bind({"weight": g2.to(dtype).cuda()}, rt)
    stream = Stream(x, a.cuda(), b.cuda(), 0.3)
    h1, h2 = n1.forward_pair(ctx, stream, n2)
    s = x.double().cpu() + 0.3 * (a.double() + b.double())
    assert stream.branch is None and stream.branch2 is None and stream.scale == 1.0 and stream.x.dtype == torch.float32
    assert (stream.x.double().cpu() - s).abs().max() < 1e-5  # the sum is 32-bit whatever the path
    close(h1.tensor(), plain.rms_norm(s, g1.double(), 1e-4), dtype, "first norm")
    close(h2.tensor(), plain.rms_norm(s, g2.double(), 1e-4), dtype, "second norm")
    only = n1.forward(ctx, Stream(x, None, b.cuda(), 2.0)).tensor()  # one pending output, in the second place
    close(only, plain.rms_norm(x.double().cpu() + 2.0 * b.double(), g1.double(), 1e-4), dtype, "one output, doubled")


ATTN_SHAPES = [  # hidden, heads, kv_heads, dim, vdim, window, keep_first, rot, base, gate, blend
    (72, 6, 3, 16, 16, 20, 5, 16, 1e4, "element", True),
    (64, 4, 1, 32, 64, 70, 66, 8, 2e4, "element", False),
    (40, 2, 2, 24, 8, 7, 1, 24, 50.0, "head", True),
    (48, 3, 1, 8, 40, 130, 64, 2, 10.0, None, True),
    (50, 3, 3, 6, 5, 3, 2, 4, 7.0, "element", True),
    (40, 10, 1, 8, 8, 90, 0, 4, 30.0, "element", False),
    (64, 4, 2, 32, 32, 70, 66, 8, 2e4, "head", True),   # kept tokens over two pages, walked before the window's pages
    (48, 4, 1, 16, 16, 200, 130, 16, 1e4, "element", False),
]


def attention_part(shape, dtype, rt, seed=0):
    from kernel_rush_kawk_b200.parts import SinkWindowAttention

    C, H, G, D, Dv, window, keep, rot, base, gate, blend = shape
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.4, "mask": {"size": window, "keep_first": keep},
         "rot": {"dims": rot, "base": base}, "v_mix": blend}
    part = SinkWindowAttention({"hidden": C, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.4, "window": window,
                                "keep_first": keep, "rot_dims": rot, "rot_base": base, "gate": gate,
                                "value_mix": "blend" if blend else None, "eps": 1e-5})
    w = {"q": rand((H * D, C), seed + 1, 0.4), "k": rand((G * D, C), seed + 2, 0.4), "v": rand((G * Dv, C), seed + 3, 0.3),
         "o": rand((C, H * Dv), seed + 4, 0.2)}
    if gate:
        w["g"] = rand((H * (Dv if gate == "element" else 1), C), seed + 5, 0.5)
    if blend:
        w["vmix"] = torch.tensor(0.37)
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    return part, m, ref


def plain_attention(h, ref, m, gate, v_first):
    """The plain mixer with the gate in the form the shape asks for (the design's own is per element)."""
    shared = {} if v_first is None else {"v_first": v_first}
    w = dict(ref)
    T, H, Dv = h.shape[0], m["heads"], m["vdim"]
    if gate == "element":
        return plain.attention(h, w, "", m, shared)
    w["g"] = torch.full((H * Dv, h.shape[1]), 0.0, dtype=torch.float64)  # sigmoid(0) = 1/2 everywhere
    w["o"] = ref["o"] * 2.0
    if gate == "head":
        o_gate = torch.sigmoid(h @ ref["g"].T).repeat_interleave(Dv, dim=1)  # [T, H * Dv]
        # the gate commutes with nothing after it, so it is folded in by hand: run with unit gate, per head
        T_ = h.shape[0]
        pos = torch.arange(T_)
        q = plain.rotate_part((h @ w["q"].T).view(T_, H, m["dim"]), pos, m["rot"]["dims"], m["rot"]["base"])
        k = plain.rotate_part((h @ w["k"].T).view(T_, m["kv_heads"], m["dim"]), pos, m["rot"]["dims"], m["rot"]["base"])
        v = (h @ w["v"].T).view(T_, m["kv_heads"], Dv)
        if v_first is not None:
            v = (1 - ref["vmix"]) * v + ref["vmix"] * v_first
        see = plain.visible(T_, m["mask"]["size"], m["mask"]["keep_first"])
        o = plain.masked_softmax_mix(q, k, v, m["scale"], see).reshape(T_, H * Dv)
        return (o * o_gate) @ ref["o"].T
    return plain.attention(h, w, "", m, shared)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", ATTN_SHAPES)
def test_attention_with_kept_tokens_gate_and_blended_values_alone(dtype, shape):
    rt = runtime(dtype)
    part, m, ref = attention_part(shape, dtype, rt)
    T = 200
    G, Dv, gate, blend = shape[2], shape[4], shape[9], shape[10]
    h = rand((T, shape[0]), 9).to(dtype)
    first = rand((T, G * Dv), 10).to(dtype) if blend else None

    def before(ctx, start, n):
        ctx.shared["value_mix"] = first[start:start + n].cuda() if blend else None

    want = plain_attention(h.double(), ref, m, gate, first.double().view(T, G, Dv) if blend else None)
    for pieces in ([T], [63, 2, 64, 71], [150] + [1] * 50):
        got = run_part(part, rt, h, pieces, dtype, before=before)
        close(got, want, dtype, f"attention {shape}, pieces {pieces[:4]}")


def test_the_first_layer_of_a_blend_leaves_its_values_for_the_others():
    rt = runtime(torch.float32)
    shape = (40, 2, 2, 8, 12, 9, 2, 4, 100.0, "element", False)
    part, m, ref = attention_part(shape, torch.float32, rt)
    part.value_mix = "first"
    h = rand((10, 40), 3)
    seen = {}

    def before(ctx, start, n):
        seen["ctx"] = ctx

    run_part(part, rt, h, [10], torch.float32, before=before)
    left = seen["ctx"].shared["value_mix"]
    close(left, h.double() @ ref["v"].T, torch.float32, "the values a first layer leaves")


LATENT_SHAPES = [  # hidden, heads, dim, vdim, rank, window, sink
    (64, 4, 16, 24, 32, None, False),
    (72, 3, 8, 40, 48, 40, True),
    (50, 3, 7, 5, 9, 4, True),
    (48, 1, 64, 16, 8, None, False),
    (64, 12, 8, 8, 96, 70, True),
    (40, 2, 12, 12, 130, 64, False),
    (64, 16, 8, 8, 512, 100, True),   # rows of 512 elements: single tokens take four query heads a block
    (40, 5, 12, 12, 260, None, False),
    (64, 4, 16, 16, 40, 50, True),    # key and value heads of one size: whole prompts in bfloat16 on the tensor cores
    (64, 2, 32, 32, 24, None, False),
]


def latent_part(shape, dtype, rt, seed=30):
    from kernel_rush_kawk_b200.parts import LatentAttention

    C, H, D, Dv, R, window, sink = shape
    m = {"heads": H, "dim": D, "vdim": Dv, "kv_rank": R, "scale": 0.3}
    part = LatentAttention({"hidden": C, "heads": H, "dim": D, "vdim": Dv, "kv_rank": R, "scale": 0.3, "window": window,
                            "sink": sink, "gate": True, "eps": 1e-5})
    w = {"q": rand((H * D, C), seed + 1, 0.4), "dkv": rand((R, C), seed + 2, 0.4), "dkv.norm": 1 + rand((R,), seed + 3, 0.2),
         "uk": rand((H * D, R), seed + 4, 0.4), "uv": rand((H * Dv, R), seed + 5, 0.3), "g": rand((H, C), seed + 6, 0.5),
         "o": rand((C, H * Dv), seed + 7, 0.2)}
    if sink:
        w["sink"] = rand((H,), seed + 8, 2.0)
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    return part, m, ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", LATENT_SHAPES)
def test_latent_attention_alone(dtype, shape):
    """Whole, in pieces down to two tokens, token by token, and in a slot that another sequence used."""
    rt = runtime(dtype)
    part, m, ref = latent_part(shape, dtype, rt)
    T = 150
    h = rand((T, shape[0]), 11).to(dtype)
    want = plain.latent_attention(h.double(), ref, "", m, 1e-5, shape[5], ref.get("sink"))
    other = rand((70, shape[0]), 12).to(dtype)
    for pieces, prior in (([T], ()), ([63, 2, 64, 21], ()), ([100] + [1] * 50, ()), ([T], [(other, [70])])):
        got = run_part(part, rt, h, pieces, dtype, prior=prior)
        close(got, want, dtype, f"latent attention {shape}, pieces {pieces[:4]}, prior {len(prior)}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_of_latent_attention_counts_once_and_has_no_value(dtype):
    rt = runtime(dtype)
    shape = (32, 2, 8, 16, 24, 12, True)
    part, m, ref = latent_part(shape, dtype, rt)
    part.sink = torch.tensor([80.0, -80.0], device="cuda")
    ref["sink"] = torch.tensor([80.0, -80.0], dtype=torch.float64)
    part._w_out = torch.eye(32, dtype=dtype, device="cuda")  # look at the heads themselves
    ref["o"] = torch.eye(32, dtype=torch.float64)
    h = rand((40, 32), 3).to(dtype)
    got = run_part(part, rt, h, [40], dtype).double().cpu()
    close(got, plain.latent_attention(h.double(), ref, "", m, 1e-5, 12, ref["sink"]), dtype, "sinks of +80 and -80")
    assert got[:, :16].abs().max() < 1e-6 and got[:, 16:].abs().max() > 0.01


EDGES = [  # window, keep_first, the loud token, total
    (10, 0, 3, 40), (64, 0, 0, 140), (65, 0, 63, 200), (300, 0, 5, 420),  # the window's own edge (also on a page border, far back)
    (10, 4, 3, 60), (10, 4, 4, 60), (20, 64, 63, 150), (20, 64, 64, 150), (7, 65, 64, 160), (7, 65, 65, 160),  # kept or not
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window, keep, loud, T", EDGES)
def test_one_loud_token_at_the_edges_of_what_a_query_sees(dtype, window, keep, loud, T):
    """One token's input is fifty times the others', so its value dominates every output that sees it: a
    window or a kept prefix that is one token off shows as a row that is loud or quiet at the wrong place.
    Whole, with the edge crossed token by token, and in pieces of two; both kinds of mixer."""
    rt = runtime(dtype)
    C = 32
    h = rand((T, C), 21, 0.3)
    h[loud] *= 50.0
    h = h.to(dtype)
    attn_shape = (C, 2, 1, 16, 16, window, keep, 4, 100.0, "element", False)
    part, m, ref = attention_part(attn_shape, dtype, rt, seed=3)
    want = plain_attention(h.double(), ref, m, "element", None)
    sees = plain.visible(T, window, keep)[:, loud]
    quiet = want[~sees & (torch.arange(T) > loud)].abs().max() if (~sees & (torch.arange(T) > loud)).any() else 0.0
    assert want[sees].abs().max() > 10 * max(float(quiet), 1e-3)  # the case shows what it is meant to
    edge = min(T - 1, max(2, loud + window - 2))
    for pieces in ([T], [edge] + [1] * (T - edge), [2] * (T // 2)):
        close(run_part(part, rt, h, pieces, dtype, step_tokens=512), want, dtype, f"attention window {window} keep {keep} loud {loud}, pieces {pieces[:3]}")
    if keep == 0:
        lat_shape = (C, 2, 8, 8, 16, window, True)
        part, m, ref = latent_part(lat_shape, dtype, rt)
        want = plain.latent_attention(h.double(), ref, "", m, 1e-5, window, ref["sink"])
        for pieces in ([T], [edge] + [1] * (T - edge), [2] * (T // 2)):
            close(run_part(part, rt, h, pieces, dtype, step_tokens=512), want, dtype, f"latent window {window} loud {loud}, pieces {pieces[:3]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [24, 33])
def test_gated_activation_with_a_gate_of_one_number_per_row(dtype, inter):
    """act(g) * u times the sigmoid of one more column of the same row (a gate that rides in the same product)."""
    rt = runtime(dtype)
    gu = rand((9, 2 * inter + 8), 2, 1.5).to(dtype)
    got = rt.ops.gated_act(gu.cuda(), inter, "silu", row_gate_col=2 * inter)
    g = gu.double()
    want = plain.silu(g[:, :inter]) * g[:, inter:2 * inter] * torch.sigmoid(g[:, 2 * inter:2 * inter + 1])
    close(got, want, dtype, "gated activation with a row gate")
    close(rt.ops.gated_act(gu.cuda(), inter, "silu"), plain.silu(g[:, :inter]) * g[:, inter:2 * inter], dtype, "without")


MOE_SHAPES = [  # hidden, experts, top, ff, shared ff
    (64, 5, 2, 40, 24), (96, 8, 1, 48, None), (50, 3, 3, 11, 7), (64, 16, 4, 32, 64), (32, 2, 2, 16, 8),
    (32, 9, 8, 1800, None),  # eight wide experts a token: their activations take the opt-in shared memory size
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", MOE_SHAPES)
@pytest.mark.parametrize("rows", [1, 5, 200])
def test_routed_experts_alone(dtype, shape, rows):
    """Few rows (every pair reads its expert) and many (rows ordered by expert) against the plain loop."""
    from kernel_rush_kawk_b200.parts import RoutedExperts

    rt = runtime(dtype)
    C, E, top, F, Fs = shape
    part = RoutedExperts({"hidden": C, "experts": E, "top": top, "intermediate": F, "shared_intermediate": Fs,
                          "shared_gate": Fs is not None})
    w = {"router": rand((E, C), 1, 0.5), "router.b": rand((E,), 2, 0.5)}
    for e in range(E):
        w.update({f"e{e}.gate": rand((F, C), 10 + 3 * e, 0.3), f"e{e}.up": rand((F, C), 11 + 3 * e, 0.3),
                  f"e{e}.down": rand((C, F), 12 + 3 * e, 0.3)})
    if Fs is not None:
        w.update({"shared.gate": rand((Fs, C), 3, 0.3), "shared.up": rand((Fs, C), 4, 0.3), "shared.down": rand((C, Fs), 5, 0.3),
                  "shared.sg": rand((1, C), 6, 0.5)})
    assert {k: tuple(s.shape) for k, s in part.tensor_specs().items()} == {k: tuple(v.shape) for k, v in w.items()}
    dev, ref = as_path(w, dtype)
    part.bind(dev, rt)
    h = rand((rows, C), 7, 1.5).to(dtype)
    mlp = {"router": {"experts": E, "top": top}, "shared": None if Fs is None else {"ff": Fs}}
    want = plain.routed_ff(h.double(), ref, "", mlp)
    for decode in (False, True):
        ctx = SimpleNamespace(ops=rt.ops, batch=SimpleNamespace(is_decode=decode))
        close(part.forward(ctx, h.cuda()), want, dtype, f"experts {shape}, {rows} rows, single-token step {decode}")


def test_routing_takes_the_lower_index_on_a_tie_and_weighs_by_the_chosen_logits_only():
    rt = runtime(torch.float32)
    x = torch.eye(4, device="cuda")
    w = torch.tensor([[1.0, 2.0, 0.0, -1.0], [3.0, 2.0, 0.0, 5.0], [3.0, 0.5, 0.0, 5.0], [0.0, 2.0, 0.0, 4.0]], device="cuda").t().contiguous()
    b = torch.zeros(4, device="cuda")
    experts, weights, _ = rt.ops.moe_route(x, w, b, 2)  # the logits of row r are column r of the table above
    z = x @ w.t()
    for r in range(4):
        best = sorted(range(4), key=lambda e: (-float(z[r, e]), e))[:2]
        assert experts[r].tolist() == best, (r, experts[r].tolist(), best)
        ref = torch.softmax(z[r, best], dim=0)
        assert torch.allclose(weights[r], ref, atol=1e-6)


# ----------------------------------------------------------------------------------------------
# the model through the engine
# ----------------------------------------------------------------------------------------------

def engine(folder, dtype, **kw):
    from kernel_rush_kawk_b200 import Engine

    args = dict(dtype=dtype, max_tokens=4096, max_slots=6, max_context=1024)
    args.update(kw)
    return Engine(folder, **args)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_portions_and_single_tokens_through_the_engine(folders, name, dtype):
    from kernel_rush_kawk_b200 import StepEntry

    eng = engine(folders[name], dtype, step_tokens=40)  # longer steps are cut into passes, and the rings turn
    ids = prompts(name, [300])[0]
    ref = plain_logits(folders[name], ids)
    for pieces in ([300], [130, 2, 3, 64, 101], [250] + [1] * 50):
        slot = eng.cache.alloc()
        got, start = [], 0
        for n in pieces:
            got.append(eng.step([StepEntry(slot, ids[start:start + n], list(range(n)))]).clone())
            start += n
        eng.cache.free(slot)
        assert_logits(torch.cat(got), ref, dtype, f"{name} {dtype}, pieces {pieces[:4]}")
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_reused_slots_and_long_decoding(folders, dtype):
    """Five requests of unequal length start together and are decoded together while the shorter ones end;
    their slots and pages are then used again by others. Every row against the sequence run alone in the
    plain implementation."""
    from kernel_rush_kawk_b200 import StepEntry

    name = "da"
    eng = engine(folders[name], dtype, max_slots=5)
    for round_ in range(2):
        lengths = [90, 1, 200, 37, 64] if round_ == 0 else [65, 130, 2]
        tails = [70, 0, 100, 20, 1] if round_ == 0 else [30, 60, 1]
        seqs = prompts(name, lengths, seed=5 + round_)
        slots = [eng.cache.alloc() for _ in seqs]
        heads = [len(ids) - t for ids, t in zip(seqs, tails)]
        first = eng.step([StepEntry(s, ids[:n], [n - 1]) for s, ids, n in zip(slots, seqs, heads)]).clone()
        for i, (ids, n) in enumerate(zip(seqs, heads)):
            assert_logits(first[i:i + 1], plain_logits(folders[name], ids)[n - 1:n], dtype, f"round {round_}, prompt {i}")
        got = {i: [] for i in range(len(seqs))}
        for t in range(max(tails)):
            live = [i for i in range(len(seqs)) if t < tails[i]]
            out = eng.step([StepEntry(slots[i], [seqs[i][heads[i] + t]], [0]) for i in live])
            for row, i in enumerate(live):
                got[i].append(out[row].clone())
            for i in range(len(seqs)):
                if t + 1 == tails[i]:
                    eng.cache.free(slots[i])
        for i, ids in enumerate(seqs):
            if tails[i] == 0:
                eng.cache.free(slots[i])
                continue
            assert_logits(torch.stack(got[i]), plain_logits(folders[name], ids)[heads[i]:], dtype, f"round {round_}, decoded sequence {i}")
        eng.cache.check()
        assert eng.cache.live == 0


def test_greedy_generation_through_the_engines_own_entry(folders):
    """Engine.generate (scheduler, captured single-token steps, selection kernel) against greedy decoding
    with the plain implementation; prompts of unequal length, one of a single token."""
    name = "db"
    eng = engine(folders[name], "float32", max_tokens=None)
    seqs = prompts(name, [33, 1, 80], seed=9)
    steps = list(eng.generate(seqs, 12))
    assert len(steps) == 12
    cfg, w = plain.read_folder(folders[name], torch.float64)
    for i, ids in enumerate(seqs):
        ids = list(ids)
        for t in range(12):
            logits = plain.forward(cfg, w, ids)[-1]
            best = torch.topk(logits, 2).values
            if best[0] - best[1] < 1e-4:  # too close to call in 32-bit: stop comparing this sequence
                break
            assert steps[t][i] == int(logits.argmax()), f"sequence {i}, new token {t}"
            ids.append(steps[t][i])


def test_trace_replay_serves_the_design(folders, tmp_path):
    """bin/trace_run's program on a small schedule: a batch of prompts, single tokens, a request that ends."""
    from kernel_rush_kawk_b200 import replay

    name = "dc"
    a, b = prompts(name, [70, 9], seed=4)
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": a[:60], "want": [0, 59]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[60]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": []}], "end": ["b"]}]
    lines += [{"step": 2 + t, "entries": [{"id": "a", "tokens": [a[61 + t]], "want": [0]}], "end": ["a"] if t == 8 else []} for t in range(9)]
    out = io.StringIO()
    args = replay.build_parser().parse_args(["--model", str(folders[name]), "--dtype", "float32", "--out", str(tmp_path / "o"),
                                             "--max-tokens", "256"])
    assert replay.run(args, stdin=io.StringIO("\n".join(json.dumps(l) for l in lines) + "\n"), stdout=out) == 0
    assert out.getvalue().split() == [w for t in range(11) for w in ("done", str(t))]
    import numpy as np
    ref_a, ref_b = plain_logits(folders[name], a), plain_logits(folders[name], b)
    first = torch.from_numpy(np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(3, -1))
    assert_logits(first, torch.stack([ref_a[0], ref_a[59], ref_b[7]]), "float32", "replayed prompts")
    for t in range(10):
        row = torch.from_numpy(np.fromfile(tmp_path / "o" / f"{1 + t}.f32", dtype="<f4").reshape(1, -1))
        assert_logits(row, ref_a[60 + t:61 + t], "float32", f"replayed token {t}")
