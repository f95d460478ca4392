"""Binupel on the GPU against the plain implementation (tests/plain_binupel.py): each mechanism alone, then
whole models in every cut, batches, reuse of pages and slots, far keys and edges made to show, long decoding and
greedy generation through the engine's entry point."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_binupel as plain
from binupel_models import CONFIGS, make_folder
from harness import Replayer, assert_close

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {key: make_folder(str(tmp_path_factory.mktemp(f"binupel_{key}")), config, seed)
            for key, (config, seed) in CONFIGS.items()}


def tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double()
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-9)
    assert err <= TOL[dtype], f"{what}: relative error {err:.3g} > {TOL[dtype]:g}"


# ---------------------------------------------------------------------- each mechanism alone
def part_weights(part, dtype, seed, scale=None):
    """Random tensors for a part's specs, strong enough to matter: (device dict, float64 copies by short name)."""
    g = torch.Generator().manual_seed(seed)
    dev, ref = {}, {}
    for s in part.weight_specs():
        leaf = s.name.split(".", 1)[1]
        if s.init == "one_plus_normal":
            t = 1 + 0.2 * torch.randn(s.shape, generator=g)
        elif len(s.shape) >= 2 and s.kind == "matrix":
            t = torch.randn(s.shape, generator=g) * (1.3 / s.shape[-1] ** 0.5)
        elif leaf == "A_log":
            t = torch.log(0.3 + 3 * torch.rand(s.shape, generator=g))
        else:
            t = 0.5 * torch.randn(s.shape, generator=g)
        if scale and leaf in scale:
            t = t * scale[leaf]
        stored = t.to(torch.bfloat16)  # what a model folder would hold
        dev[s.name] = stored.to(torch.float32 if s.kind == "vector" else DT[dtype]).cuda()
        ref[leaf] = stored.double()
    return dev, ref


class MixerBench:
    """One mixer (or block) with a cache manager, storage and batches of its own."""

    def __init__(self, part, dtype, page_size=4, pages=96, max_tokens=512, max_seqs=3, seed=0, scale=None, tweak=None):
        from qwen3_from_scratch_b200.cache import CacheManager, layout_of
        from qwen3_from_scratch_b200.cache.storage import CacheStorage
        from qwen3_from_scratch_b200.parts.base import Runtime
        self.part, self.dtype = part, dtype
        self.rt = Runtime(torch.device("cuda:0"), DT[dtype], max_tokens, max_seqs)
        self.dev, self.ref = part_weights(part, dtype, seed, scale)
        if tweak is not None:
            tweak(self.dev, self.ref)
        part.setup(self.rt, dict(self.dev))
        layout = layout_of({0: part.cache_spec()})
        self.manager = CacheManager(layout, page_size, pages, max_seqs)
        self.storage = CacheStorage(layout, page_size, max_seqs, self.rt.device, self.rt.dtype)
        self.manager.on_open = self.storage.clear_slot

    def run(self, portions, x_of, call):
        """``portions``: [(request, count)] of one step; feeds x_of[request] rows on; returns outputs by request."""
        from qwen3_from_scratch_b200.engine.batch import BatchContext, Entry
        entries = []
        for req, n in portions:
            if req not in self.manager:
                self.manager.open(req)
            self.manager.reserve(req, self.manager.length(req) + n)
            entries.append(Entry(req, [0] * n))
        ctx = BatchContext(self.manager, self.storage, self.rt).build(entries, vocab_size=1)
        rows = {r: i for i, r in enumerate(ctx.requests)}
        x = torch.cat([x_of[r][self.manager.length(r):self.manager.length(r) + self.rows_of(portions, r)]
                       for r in ctx.requests])
        y = call(x, ctx)
        out, starts = {}, ctx.q_start.cpu().tolist()
        for req, n in portions:
            b = rows[req]
            out[req] = y[starts[b]:starts[b + 1]].clone()
            self.manager.advance(req, self.manager.length(req) + n)
        assert int(self.rt.status.item()) == 0
        return out

    @staticmethod
    def rows_of(portions, req):
        return dict(portions)[req]


MIXERS = {
    "sigmoid_attention": ({"hidden_size": 40, "num_heads": 6, "num_kv_heads": 2, "head_dim": 32, "scale": 0.25,
                           "qk_norm_eps": 1e-5, "temp_coef": 0.7, "temp_every": 5},
                          lambda h, ref, st: plain.sigmoid_attention(
                              h, ref, "", {"heads": 6, "kv_heads": 2, "dim": 32, "scale": 0.25,
                                           "q_temp": {"coef": 0.7, "every": 5}}, 1e-5, st)),
    "rglru": ({"hidden_size": 40, "width": 72, "blocks": 3, "conv": 4},
              lambda h, ref, st: plain.rglru(h, ref, "", 3, st)),
    "selective_scan": ({"hidden_size": 40, "inner": 56, "state": 12, "dt_rank": 6, "conv": 3},
                       lambda h, ref, st: plain.selective_scan(h, ref, "", 6, st)),
    # the edges of the sizes: a single tap (no tail to keep), one block of gates, an odd channel count; a state
    # beyond 32, a step rank of 3, five taps (beyond the convolution kernel that is compiled per number of taps)
    "rglru, one tap": ({"hidden_size": 40, "width": 44, "blocks": 1, "conv": 1},
                       lambda h, ref, st: plain.rglru(h, ref, "", 1, st)),
    "selective_scan, wide state": ({"hidden_size": 40, "inner": 24, "state": 40, "dt_rank": 3, "conv": 5},
                                   lambda h, ref, st: plain.selective_scan(h, ref, "", 3, st)),
}


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("kind", list(MIXERS))
def test_mixer_alone_whole_in_portions_and_beside_another_request(kind, dtype):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    params, plain_fn = MIXERS[kind]
    bench = MixerBench(create_part("mixer", PartSpec(kind.split(",")[0], params), name="m"), dtype, seed=11)
    g = torch.Generator().manual_seed(12)
    x_of = {r: torch.randn(n, 40, generator=g).to(DT[dtype]) for r, n in (("a", 41), ("b", 19))}
    want = {r: plain_fn(x.double(), bench.ref, None)[0] for r, x in x_of.items()}
    call = lambda x, ctx: bench.part.forward(x.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    # whole, each alone
    for r in x_of:
        close(bench.run([(r, len(x_of[r]))], x_of, call)[r], want[r], dtype, f"{kind} whole {r}")
        bench.manager.close(r)
    # portions down to one and two tokens, the second request joining and leaving in between
    got = {r: [] for r in x_of}
    for step in ([("a", 7)], [("a", 1)], [("a", 2), ("b", 2)], [("b", 1), ("a", 1)], [("a", 13), ("b", 16)],
                 [("a", 2)], [("a", 1)], [("a", 14)]):
        for r, y in bench.run(step, x_of, call).items():
            got[r].append(y)
    for r in x_of:
        close(torch.cat(got[r]), want[r], dtype, f"{kind} portions {r}")


@pytest.mark.parametrize("kind", ["rglru", "selective_scan"])
def test_long_portions_run_in_chunks_and_leave_the_same_state(kind):
    """bfloat16: a portion of several hundred tokens is cut into chunks that run side by side, a short one is
    walked by one thread per channel; a long portion beside a single token of another request, then the same
    tokens in short portions: the outputs agree with the plain implementation and the float32 states that the
    two ways leave agree to float32 rounding."""
    from qwen3_from_scratch_b200.kernels import ops
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    params, plain_fn = MIXERS[kind]
    bench = MixerBench(create_part("mixer", PartSpec(kind, params), name="m"), "bfloat16", max_tokens=1024, pages=8, seed=13)
    g = torch.Generator().manual_seed(14)
    x_of = {"a": torch.randn(700, 40, generator=g).to(torch.bfloat16), "b": torch.randn(3, 40, generator=g).to(torch.bfloat16)}
    want = {r: plain_fn(x.double(), bench.ref, None)[0] for r, x in x_of.items()}
    call = lambda x, ctx: bench.part.forward(x.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    assert ops.scan_chunked_pays(torch.bfloat16, 697) and not ops.scan_chunked_pays(torch.bfloat16, 100)
    states = []
    for steps in ([[("b", 2)], [("a", 697), ("b", 1)], [("a", 3)]],
                  [[("b", 2)]] + [[("a", 100)]] * 3 + [[("a", 100), ("b", 1)]] + [[("a", 100)]] * 3):
        got = {r: [] for r in x_of}
        for step in steps:
            for r, y in bench.run(step, x_of, call).items():
                got[r].append(y)
        for r in x_of:
            close(torch.cat(got[r]), want[r], "bfloat16", f"{kind} {r}")
        slot = bench.manager.slot("a")
        states.append({k: t[slot].clone() for k, t in bench.storage.states.items()})
        bench.manager.close("a")
        bench.manager.close("b")
    for k in states[0]:
        scale = float(states[0][k].abs().max())
        assert float((states[0][k] - states[1][k]).abs().max()) <= 2e-5 * scale, k


@pytest.mark.parametrize("dtype", list(DT))
def test_post_norm_block_with_shift_and_relu_gate(dtype):
    """The block's arrangement: shift on the mixer's input only, alpha on the stream, the norm after each sum, the
    feed-forward on the normed stream; cut between any two tokens."""
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    W = 40
    norm = PartSpec("rms_norm", {"dim": W, "eps": 1e-5, "suffix": ""})
    block = create_part("block", PartSpec("post_norm", {
        "norm1": norm, "norm2": norm, "alpha": 1.7, "token_shift": True, "width": W,
        "mixer": PartSpec("rglru", {"hidden_size": W, "width": 48, "blocks": 2, "conv": 2}),
        "feed_forward": PartSpec("gated_mlp", {"hidden_size": W, "intermediate_size": 56, "activation": "relu",
                                               "names": {"gate": "gate", "up": "up", "down": "down"}}),
        "names": {"mixer": "mix", "feed_forward": "mlp"}}), name="l0")
    bench = MixerBench(block, dtype, seed=21)
    config = {"norm": {"eps": 1e-5}, "postln_alpha": 1.7,
              "layers": [{"type": "rglru", "mixer": {"blocks": 2}, "mlp": {"kind": "dense"}}]}
    w = {"l0." + k: v for k, v in bench.ref.items()}
    x = torch.randn(17, W, generator=torch.Generator().manual_seed(22))
    want = plain.layer(x.double(), w, config, 0)[0]

    def call(rows, ctx):
        stream = rows.float().cuda().contiguous()
        assert block.forward(stream, None, ctx, 0, True) is None
        return stream

    for cuts in ([17], [1, 1, 2, 5, 1, 7]):
        got = [bench.run([("r", c)], {"r": x}, call)["r"] for c in cuts]
        bench.manager.close("r")
        close(torch.cat(got), want, dtype, f"block {cuts}")


@pytest.mark.parametrize("rows", [3, 12, 40, 200, 1100])
def test_relu_gated_feed_forward_in_every_product(rows):
    """bfloat16: the gate is applied by the few-rows product (up to 16 rows), by the tcgen05 product's epilogue
    (single CTAs from 128 rows, pairs from 1,024) or by the gate kernel after the library's product."""
    from qwen3_from_scratch_b200.parts.base import PartSpec, Runtime
    from qwen3_from_scratch_b200.registry import create_part
    part = create_part("feed_forward", PartSpec("gated_mlp", {
        "hidden_size": 128, "intermediate_size": 256, "activation": "relu",
        "names": {"gate": "gate", "up": "up", "down": "down"}}), name="f")
    dev, ref = part_weights(part, "bfloat16", 23)
    part.setup(Runtime(torch.device("cuda:0"), torch.bfloat16, 2048, 2), dev)
    x = torch.randn(rows, 128, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16)
    close(part.forward(x.cuda()), plain.relu_glu(x.double(), ref, ""), "bfloat16", f"{rows} rows")


def test_shift_state_is_the_input_before_the_shift():
    """mu = 1 makes the mixer read the previous token's x alone: the second token of a request, fed alone, must
    see the first one's stream, not the first one's shifted input."""
    from qwen3_from_scratch_b200.kernels import ops
    W = 8
    x = torch.arange(3 * W, dtype=torch.float32).view(3, W).cuda() + 1
    state = torch.zeros(2, W, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mu = torch.ones(W, device="cuda")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    out = torch.empty(2, W, device="cuda")
    ops.token_shift(x[:2].contiguous(), mu, state, i32([0, 2]), i32([0, 0]), i32([1]), out, status)
    assert torch.equal(out[0], torch.zeros(W, device="cuda")) and torch.equal(out[1], x[0])
    assert torch.equal(state[1], x[1]) and not state[0].any()
    out1 = torch.empty(1, W, device="cuda")
    ops.token_shift(x[2:].contiguous(), mu, state, i32([0, 1]), i32([0]), i32([1]), out1, status)
    assert torch.equal(out1[0], x[1]) and torch.equal(state[1], x[2])


# ---------------------------------------------------------------------- far keys and the causal edge
@pytest.mark.parametrize("dtype", list(DT))
def test_one_far_key_decides_the_output(dtype):
    """A strongly negative head bias closes every key; one key far back (at a page's last slot, hundreds of
    tokens before the query) is opened by a large score against chosen queries.  Those queries' outputs are that
    key's value times the gate, every other query's is nearly nothing; as a prompt's portion and decoded alone."""
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    W, H, G, d, page, n, far = 32, 4, 2, 64, 16, 420, 47
    part = create_part("mixer", PartSpec("sigmoid_attention", {
        "hidden_size": W, "num_heads": H, "num_kv_heads": G, "head_dim": d, "scale": 1.0, "qk_norm_eps": 1e-6}), name="m")

    def tweak(dev, ref):
        # a query head's projection is its kv head's key projection: equal inputs give parallel q and k, whose
        # normed product is about d; unrelated inputs give about sqrt(d); the bias lies between the two
        for tensors, pre in ((dev, "m."), (ref, "")):
            k = tensors[pre + "k"].view(G, d, W)
            tensors[pre + "q"].copy_(k.repeat_interleave(H // G, dim=0).reshape(H * d, W))
            tensors[pre + "pb"].fill_(-40.0)

    bench = MixerBench(part, dtype, page_size=page, pages=64, max_tokens=512, seed=31, tweak=tweak)
    # inputs: small noise everywhere; the far token and the asking tokens carry a large common direction
    g = torch.Generator().manual_seed(32)
    x = 0.05 * torch.randn(n, W, generator=g)
    mark = torch.randn(W, generator=g)
    askers = [far, far + 1, 200, 419]  # the key itself (the edge: n == p is visible), its neighbour, two far queries
    for t in askers:
        x[t] += 3 * mark
    x = x.to(DT[dtype])
    m = {"heads": H, "kv_heads": G, "dim": d, "scale": 1.0}
    want = plain.sigmoid_attention(x.double(), bench.ref, "", m, 1e-6)[0]
    strong = want.abs().max(dim=1).values
    # (an unmarked token still sees itself: its own key is parallel to its query, but its value is small)
    assert float(strong[askers].min()) > 20 * float(strong[[far - 1, 100, 300]].max()), "the test's weights do not single the key out"
    call = lambda rows, ctx: part.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    got = bench.run([("r", n)], {"r": x}, call)["r"]
    close(got, want, dtype, "whole prompt")
    bench.manager.close("r")
    pieces = [bench.run([("r", c)], {"r": x}, call)["r"] for c in [far, 1, 1, 150, 1] + [2] * 60 + [1] * (n - far - 273)]
    close(torch.cat(pieces), want, dtype, "portions and single tokens")


# ---------------------------------------------------------------------- the tensor-core kernel against the plain one
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 16, 4), (6, 1, 48, 16), (8, 2, 64, 16), (8, 1, 128, 16), (4, 4, 128, 8),
                                           (6, 2, 64, 32), (16, 1, 256, 8), (20, 1, 32, 16)])
def test_tensor_core_sigmoid_attention_equals_the_plain_kernel(hq, hkv, d, page):
    """A mixed batch: three single tokens at contexts that end just before, at and just after a tile's and a page's
    edge, and two portions (one from position 0, one continuing); key ranges of the decode form from 1 to many.
    (A group of more than 16 heads has no decode form: its single tokens run as portions of one.)"""
    from qwen3_from_scratch_b200.kernels import ops
    g = torch.Generator().manual_seed(41)
    q_lens, kv_lens = [1, 1, 1, 37, 150], [64, 65, 449, 37, 333]
    B, T = len(q_lens), sum(q_lens)
    pages_per = [-(-n // page) for n in kv_lens]
    num_pages = sum(pages_per) + 3
    order = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(pages_per):
        table[b, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    k_pages = torch.randn(num_pages, hkv, page, d, generator=g).to(torch.bfloat16).cuda()
    v_pages = torch.randn(num_pages, hkv, page, d, generator=g).to(torch.bfloat16).cuda()
    q = (2 * torch.randn(T, hq, d, generator=g)).to(torch.bfloat16).cuda()
    bias = torch.randn(hq, generator=g).cuda() - 3
    gate = torch.rand(T, hq, generator=g).cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    q_start = i32([0] + torch.tensor(q_lens).cumsum(0).tolist())
    tok_seq = i32([b for b, n in enumerate(q_lens) for _ in range(n)])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = (q, k_pages, v_pages)
    rest = (bias, gate, q_start, i32(kv_lens), tok_seq, table.cuda(), B, 3, max(q_lens), max(kv_lens), d ** -0.5, status)
    want = torch.empty_like(q)
    ops.sigmoid_attention(*args, want, *rest, kernel="plain")
    scale = float(want.float().abs().max())
    # the portions on mma.sync with 0, 2 and as many key ranges of the decode form as it likes, then on tcgen05
    for partial_floats, kernel in ((0, "mma"), (3 * 2 * hq * d, "mma"), (ops.sigmoid_partial_numel(3, hq, d), "mma"),
                                   (ops.sigmoid_partial_numel(3, hq, d), "auto")):
        partial = torch.empty(partial_floats, device="cuda") if partial_floats else None
        got = torch.full_like(q, float("nan"))
        ops.sigmoid_attention(*args, got, *rest, partial=partial, kernel=kernel)
        assert int(status.item()) == 0
        # both round the weights' sum to bfloat16 once; the tensor-core kernels also round each weight
        assert float((got.float() - want.float()).abs().max()) <= 1.5e-2 * scale, (partial_floats, kernel)


# ---------------------------------------------------------------------- whole models
def tolerance(dtype, cfg, w, seqs):
    """float32: the harness's bound.  bfloat16: three times what rounding alone does to these prompts in the plain
    implementation (projections' operands and results rounded to bfloat16), and no less than the harness's bound;
    these small models with weights of order one amplify a rounding more than trained ones do."""
    if dtype == "float32":
        return None
    return max(TOL[dtype], 3 * max(plain.rounding_error(cfg, w, ids) for ids in seqs.values()))


def replay(folder, dtype, seqs, schedule, **session_args):
    from qwen3_from_scratch_b200.engine.session import Session
    args = dict(page_size=8, num_pages=96, max_seqs=3, max_step_tokens=256)
    args.update(session_args)
    session = Session(folder, dtype=dtype, **args)
    r = Replayer(session, seqs)
    schedule(r)
    session.manager.check()
    assert session.manager.free_slots() == args["max_seqs"]
    return r.result()


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("key", list(CONFIGS))
def test_model_whole_decoded_and_in_portions(folders, key, dtype):
    cfg, w = plain.read_model_folder(folders[key])
    ids = tokens(cfg["vocab"], 90, 51)
    want = {"a": plain.forward_logits(cfg, w, ids)}
    tol = tolerance(dtype, cfg, w, {"a": ids})

    def whole(r):
        r.step([("a", 90)])

    def decoded(r):
        r.step([("a", 50)])
        for _ in range(40):
            r.step([("a", 1)])

    def portions(r):
        for n in [3, 2, 2, 1, 17, 2, 31, 1, 1, 2, 16, 2, 8, 2]:
            r.step([("a", n)])

    for name, schedule in (("whole", whole), ("decoded", decoded), ("portions", portions)):
        assert_close(replay(folders[key], dtype, {"a": ids}, schedule), want, dtype, f"{key} {name}", tol=tol)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("key", ["p", "r"])
def test_unequal_requests_together_equal_each_alone_with_pages_and_slots_used_again(folders, key, dtype):
    """Five requests through two state slots and a pool that holds less than their sum: portions of some beside
    single tokens of others; a slot and its pages go to the next request as soon as one ends; freed pages are
    filled with NaN."""
    cfg, w = plain.read_model_folder(folders[key])
    lens = {"a": 61, "b": 7, "c": 33, "d": 1, "e": 40}
    seqs = {r: tokens(cfg["vocab"], n, 60 + i) for i, (r, n) in enumerate(lens.items())}
    want = {r: plain.forward_logits(cfg, w, ids) for r, ids in seqs.items()}

    def schedule(r):
        r.step([("a", 30), ("b", 5)])
        r.step([("a", 1), ("b", 2)])             # b ends: its slot is free
        r.step([("c", 2), ("a", 1)])             # c takes b's slot
        r.step([("a", 1), ("c", 20)])
        r.step([("c", 1)])                       # a is left out of a step
        r.step([("a", 28), ("c", 10)])           # both end
        r.step([("d", 1), ("e", 9)])             # a request of a single token
        for _ in range(31):
            r.step([("e", 1)])

    got = replay(folders[key], dtype, seqs, schedule, page_size=4, num_pages=26, max_seqs=2, poison_freed_pages=True)
    assert_close(got, want, dtype, f"{key} mixed", tol=tolerance(dtype, cfg, w, seqs))


def test_long_prompt_on_the_serving_kernels(folders):
    """bfloat16, heads of 64 and 128 with pages of 16: a prompt of 700 tokens whole (several tiles of the tcgen05
    portion attention, the scans in chunks, the tcgen05 gate/up product) and cut into long and short portions with
    single tokens between them."""
    cfg, w = plain.read_model_folder(folders["r"])
    ids = tokens(cfg["vocab"], 700, 77)
    want = {"a": plain.forward_logits(cfg, w, ids)}
    tol = tolerance("bfloat16", cfg, w, {"a": ids})
    for name, cuts in (("whole", [700]), ("portions", [300, 1, 250, 1, 1, 130, 17])):
        got = replay(folders["r"], "bfloat16", {"a": ids}, lambda r, cuts=cuts: [r.step([("a", n)]) for n in cuts],
                     page_size=16, num_pages=64, max_seqs=2, max_step_tokens=1024)
        assert_close(got, want, "bfloat16", f"r long {name}", tol=tol)


def test_long_decoding_through_graphs(folders):
    """300 single tokens after a short prompt, replayed from CUDA graphs: the states are carried on the device
    from step to step; the last logits still agree with the plain implementation in float32."""
    cfg, w = plain.read_model_folder(folders["q"])
    ids = tokens(cfg["vocab"], 310, 71)
    want = {"a": plain.forward_logits(cfg, w, ids)}

    def schedule(r):
        r.step([("a", 10)])
        for _ in range(300):
            r.step([("a", 1)])

    got = replay(folders["q"], "float32", {"a": ids}, schedule, num_pages=64, max_seqs=2)
    assert_close(got, want, "float32", "long decoding")


def test_float32_cuts_give_identical_bits(folders):
    """In float32 every sum has an order that depends only on the token, so a prompt whole, in portions and
    token by token gives the same bits."""
    cfg, _ = plain.read_model_folder(folders["p"])
    ids = tokens(cfg["vocab"], 45, 81)
    runs = [replay(folders["p"], "float32", {"a": ids}, s)["a"] for s in (
        lambda r: r.step([("a", 45)]),
        lambda r: [r.step([("a", n)]) for n in (7, 2, 1, 20, 15)],
        lambda r: [r.step([("a", 1)]) for _ in range(45)])]
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])


# ---------------------------------------------------------------------- the engine's entry points
@pytest.mark.parametrize("key", ["p", "q"])
def test_greedy_generation_through_the_engine_equals_plain(folders, key):
    """Prompts of unequal length through SyncEngine.batch_generate: chunked prompts, continuous batching with
    fewer slots than requests, lookahead, CUDA graphs; float32, prompts chosen so that no step is a near tie."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    cfg, w = plain.read_model_folder(folders[key])
    prompts, expected = [], []
    for i, n in enumerate([1, 9, 33, 70]):
        for seed in range(100 * i, 100 * i + 50):
            prompt = tokens(cfg["vocab"], n, seed)
            out, margins = plain.greedy(cfg, w, prompt, 12)
            if min(margins) > 1e-3:
                break
        prompts.append(prompt)
        expected.append(out)
    engine = SyncEngine(folders[key], dtype="float32", block_size=8, num_pages=64, max_num_seqs=3, max_num_tokens=48,
                        chunked_prefill_size=16)
    results, batch = engine.batch_generate(prompts, max_new_tokens=12, ignore_eos=True)
    assert batch.num_requests == 4
    for want, r in zip(expected, results):
        assert r.token_ids == want and r.finish_reason == "length"
    engine.session.manager.check()
    assert engine.session.manager.free_slots() == 3


def test_preempted_request_is_recomputed_from_a_clean_state(folders):
    """A pool too small for all requests at once: the one that loses its pages starts again in a zeroed slot and
    still generates what it generates alone."""
    from qwen3_from_scratch_b200.engine.engine import SyncEngine
    cfg, _ = plain.read_model_folder(folders["p"])
    prompts = [tokens(cfg["vocab"], n, 90 + i) for i, n in enumerate([30, 28, 26])]
    alone = SyncEngine(folders["p"], dtype="float32", block_size=4, num_pages=64, max_num_seqs=4, max_num_tokens=64)
    want = [alone.generate(p, max_new_tokens=24, ignore_eos=True) for p in prompts]
    tight = SyncEngine(folders["p"], dtype="float32", block_size=4, num_pages=34, max_num_seqs=4, max_num_tokens=64)
    results, _ = tight.batch_generate(prompts, max_new_tokens=24, ignore_eos=True)
    assert [r.token_ids for r in results] == want
    assert tight.scheduler.num_preemptions > 0


@pytest.mark.parametrize("dtype", list(DT))
def test_trace_replay_program_and_command_line(folders, tmp_path, dtype):
    folder = folders["q"]
    cfg, w = plain.read_model_folder(folder)
    vocab = cfg["vocab"]
    a, b = tokens(vocab, 70, 31), tokens(vocab, 50, 32)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:2], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[40:41], "want": [0]},
                                {"id": "b", "tokens": b[2:50], "want": [47, 0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[41:70], "want": list(range(29))}], "end": ["a"]},
    ]
    out = str(tmp_path / "out")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
           "--max-tokens", "192", "--poison-freed-pages"]
    proc = subprocess.run(cmd, input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(4)]
    la, lb = plain.forward_logits(cfg, w, a), plain.forward_logits(cfg, w, b)

    tol = tolerance(dtype, cfg, w, {"a": a, "b": b}) or TOL[dtype]

    def check(step, rows):
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4")).view(len(rows), vocab)
        want = torch.stack(rows)
        assert float((got - want).abs().max()) <= tol * float(max(la.abs().max(), lb.abs().max()))

    check(0, [la[0], la[39]])
    check(2, [la[40], lb[49], lb[2]])
    check(3, [la[41 + i] for i in range(29)])
    if dtype == "float32":
        prompt = a[:9]
        want, margins = plain.greedy(cfg, w, prompt, 6)
        gen = [sys.executable, "-m", "qwen3_from_scratch_b200", "generate", "--model", folder, "--dtype", "float32",
               "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6", "--ignore-eos",
               "--block-size", "4", "--num-pages", "32", "--max-num-seqs", "2", "--max-num-tokens", "32"]
        proc = subprocess.run(gen, capture_output=True, text=True, cwd=ROOT, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        if min(margins) > 1e-3:
            assert json.loads(proc.stdout.splitlines()[0])["token_ids"] == want
