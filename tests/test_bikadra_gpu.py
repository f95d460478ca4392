"""Bikadra on the GPU against the plain implementation (tests/plain_bikadra.py): the small kernels against float32
torch, each mechanism alone, then whole models in every cut, batches, reuse of pages and slots, far keys made to
show, long decoding and greedy generation through the engine's entry point."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_bikadra as plain
from bikadra_models import CONFIGS, make_folder
from harness import Replayer, assert_close
from test_binupel_gpu import MixerBench, part_weights

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {key: make_folder(str(tmp_path_factory.mktemp(f"bikadra_{key}")), config, seed)
            for key, (config, seed) in CONFIGS.items()}


def tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def close(got, want, dtype, what="", tol=None):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-9)
    bound = TOL[dtype] if tol is None else tol
    assert err <= bound, f"{what}: relative error {err:.3g} > {bound:g}"


# ---------------------------------------------------------------------- the small kernels against float32 torch
@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("S,W,T", [(1, 48, 5), (2, 64, 33), (3, 200, 7), (4, 1024, 19), (8, 96, 3), (2, 50, 4), (3, 201, 6),
                                   (2, 5000, 3)])
def test_stream_kernels(S, W, T, dtype):
    """Reading S streams into a norm with and without an open write, and the last norm over chosen rows."""
    from qwen3_from_scratch_b200.kernels import ops
    g = torch.Generator().manual_seed(S * 100 + W)
    xs = torch.randn(T, S, W, generator=g).cuda()
    delta = torch.randn(T, W, generator=g).to(DT[dtype]).cuda()
    mix = (torch.eye(S) + 0.3 * torch.randn(S, S, generator=g)).cuda()
    write, read = torch.randn(S, generator=g).cuda(), torch.randn(S, generator=g).cuda()
    weight = (1 + 0.2 * torch.randn(W, generator=g)).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    eps = 1e-5

    def norm(u):
        return u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + eps) * weight

    # no write open: the streams stay, the output is the norm of the weighted sum
    out, before = torch.empty(T, W, dtype=DT[dtype], device="cuda"), xs.clone()
    ops.hc_norm(xs, None, read, weight, out, eps, status)
    assert torch.equal(xs, before)
    close(out, norm(torch.einsum("s,tsw->tw", read, xs)), dtype, "read", tol=1e-5 if dtype == "float32" else 8e-3)
    # an open write: every stream from the old ones, mix indexed [from, to]
    new = torch.einsum("ft,xfw->xtw", mix, before) + write[None, :, None] * delta.float()[:, None, :]
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device="cuda")
    last = torch.empty(3, W, dtype=DT[dtype], device="cuda")
    ops.hc_sum_norm_rows(xs, (delta, mix, write), weight, rows, last, eps, status)
    assert torch.equal(xs, before), "the last norm must leave the streams alone"
    close(last, norm(new.sum(1))[rows.long()], dtype, "last norm", tol=1e-5 if dtype == "float32" else 8e-3)
    ops.hc_norm(xs, (delta, mix, write), read, weight, out, eps, status)
    close(xs, new, "float32", "write", tol=1e-6)
    close(out, norm(torch.einsum("s,tsw->tw", read, new)), dtype, "write then read", tol=1e-5 if dtype == "float32" else 8e-3)
    ops.hc_sum_norm_rows(xs, None, weight, rows, last, eps, status)
    close(last, norm(new.sum(1))[rows.long()], dtype, "last norm, nothing open", tol=1e-5 if dtype == "float32" else 8e-3)
    assert int(status.item()) == 0


def test_scaled_embedding_softcap_and_activation():
    from qwen3_from_scratch_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    table = torch.randn(50, 40, generator=g).to(torch.bfloat16).cuda()
    ids = torch.tensor([7, 0, 49, 7], dtype=torch.int32, device="cuda")
    out = torch.empty(4, 3, 40, device="cuda")
    ops.embed_scaled(table, ids, out, 2.5, status)
    assert torch.equal(out, (table[ids.long()].float() * 2.5)[:, None, :].expand(4, 3, 40)) and int(status.item()) == 0
    ops.embed_scaled(table, torch.tensor([50, 1, 2, 3], dtype=torch.int32, device="cuda"), out, 1.0, status)
    assert int(status.item()) == 1 and float(out[0].abs().max()) == 0  # a token outside the table is flagged, not read
    logits = (40 * torch.randn(5, 333, generator=g)).cuda()
    want = 30.0 * torch.tanh(logits / 30.0)
    ops.softcap(logits, 30.0)
    assert float((logits - want).abs().max()) < 1e-5
    for dtype, n in ((torch.float32, 77), (torch.bfloat16, 77), (torch.bfloat16, 4096)):
        x = (2 * torch.randn(3, n, generator=g)).to(dtype).cuda()
        y = torch.empty_like(x)
        ops.act(x, y, "gelu_tanh")
        close(y, plain.gelu_tanh(x.double()), "float32" if dtype == torch.float32 else "bfloat16", "gelu",
              tol=1e-6 if dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("I,parts", [(48, 1), (96, 3), (512, 2), (40, 40), (6000, 2)])
def test_gated_norm_in_parts(I, parts, dtype):
    from qwen3_from_scratch_b200.kernels import ops
    g = torch.Generator().manual_seed(I)
    y = torch.randn(9, I, generator=g).cuda()
    z = torch.randn(9, I + 10, generator=g).to(DT[dtype]).cuda()
    weight = (1 + 0.2 * torch.randn(I, generator=g)).cuda()
    out = torch.empty(9, I, dtype=DT[dtype], device="cuda")
    ops.gated_group_norm(y, z, 4, weight, out, parts, 1e-5)
    v = y.double() * plain.silu(z[:, 4:4 + I].double())
    want = plain.unit_rms(v.view(9, parts, I // parts), 1e-5).reshape(9, I) * weight.double()
    close(out, want, dtype, "gated norm", tol=1e-5 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("rows", [3, 12, 40, 300])
def test_dense_feed_forward_in_every_product(rows, dtype):
    """W_down gelu_tanh(W_up x): a few rows (the activation in the few-rows product's epilogue) and many."""
    from qwen3_from_scratch_b200.parts.base import PartSpec, Runtime
    from qwen3_from_scratch_b200.registry import create_part
    part = create_part("feed_forward", PartSpec("dense_mlp", {"hidden_size": 64, "intermediate_size": 136,
                                                              "activation": "gelu_tanh", "names": {"up": "up", "down": "down"}}),
                       name="f")
    dev, ref = part_weights(part, dtype, seed=rows)
    part.setup(Runtime(torch.device("cuda:0"), DT[dtype], 512, 2), dict(dev))
    x = torch.randn(rows, 64, generator=torch.Generator().manual_seed(rows + 1)).to(DT[dtype])
    want = plain.dense_ff(x.double(), ref, "")
    close(part.forward(x.cuda()), want, dtype, f"dense feed-forward, {rows} rows")


# ---------------------------------------------------------------------- each mixer alone
def _latent(params):
    m = {"heads": params["num_heads"], "dim": params["dim"], "rot_dim": params["rot_dim"], "vdim": params["vdim"],
         "kv_rank": params["kv_rank"], "scale": params["scale"],
         "rot": {"dims": params["position"].params["dims"], "base": params["position"].params["base"],
                 "scaling": params["position"].params["scaling"]}}
    return lambda h, ref, st: plain.latent_attention(h, ref, "", m, params["norm_eps"], st)


def _ssd(params):
    m = {"heads": params["num_heads"], "vdim": params["vdim"], "state": params["state"], "groups": params["groups"],
         "norm_groups": params["norm_groups"]}
    return lambda h, ref, st: plain.mamba2(h, ref, "", m, params["norm_eps"], st)


def mixers():
    from qwen3_from_scratch_b200.parts.base import PartSpec

    def rot(dims, base, scaling=None):
        return PartSpec("rotary_stretched", {"dims": dims, "base": base, "scaling": scaling})

    stretch = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    table = {
        "latent_attention": {"hidden_size": 40, "num_heads": 5, "dim": 24, "rot_dim": 16, "vdim": 8, "kv_rank": 40,
                             "q_rank": 24, "scale": 0.3, "norm_eps": 1e-5, "position": rot(16, 10000.0, stretch)},
        # one head, a latent wider than a warp's single pass, part of the rotated values not rotated, no stretching
        "latent_attention, one head": {"hidden_size": 40, "num_heads": 1, "dim": 8, "rot_dim": 32, "vdim": 48,
                                       "kv_rank": 72, "q_rank": 16, "scale": 0.2, "norm_eps": 1e-6,
                                       "position": rot(24, 300.0)},
        # seventeen heads (more than a tensor-core tile's sixteen rows)
        "latent_attention, many heads": {"hidden_size": 40, "num_heads": 17, "dim": 16, "rot_dim": 16, "vdim": 16,
                                         "kv_rank": 32, "q_rank": 32, "scale": 0.25, "norm_eps": 1e-5,
                                         "position": rot(16, 10000.0, stretch)},
        "ssd": {"hidden_size": 40, "num_heads": 6, "vdim": 8, "state": 24, "groups": 3, "norm_groups": 2, "conv": 4,
                "norm_eps": 1e-5},
        # one group, one norm part, a single tap, a state that one lane holds
        "ssd, one of each": {"hidden_size": 40, "num_heads": 3, "vdim": 16, "state": 8, "groups": 1, "norm_groups": 1,
                             "conv": 1, "norm_eps": 1e-6},
        # heads whose channels are no multiple of four (a channel per thread), a state of 20, five norm parts
        "ssd, odd channels": {"hidden_size": 40, "num_heads": 3, "vdim": 10, "state": 20, "groups": 3, "norm_groups": 5,
                              "conv": 2, "norm_eps": 1e-5},
        # a state spread over eight lanes, as many groups as heads, five taps
        "ssd, wide state": {"hidden_size": 40, "num_heads": 2, "vdim": 12, "state": 100, "groups": 2, "norm_groups": 3,
                            "conv": 5, "norm_eps": 1e-5},
    }
    return {k: (v, (_latent if k.startswith("latent") else _ssd)(v)) for k, v in table.items()}


MIXER_KINDS = ["latent_attention", "latent_attention, one head", "latent_attention, many heads", "ssd",
               "ssd, one of each", "ssd, wide state", "ssd, odd channels"]


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("kind", MIXER_KINDS)
def test_mixer_alone_whole_in_portions_and_beside_another_request(kind, dtype):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    params, plain_fn = mixers()[kind]
    bench = MixerBench(create_part("mixer", PartSpec(kind.split(",")[0], params), name="m"), dtype, seed=11)
    g = torch.Generator().manual_seed(12)
    x_of = {r: torch.randn(n, 40, generator=g).to(DT[dtype]) for r, n in (("a", 41), ("b", 19))}
    want = {r: plain_fn(x.double(), bench.ref, None)[0] for r, x in x_of.items()}
    call = lambda x, ctx: bench.part.forward(x.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    for r in x_of:  # whole, each alone
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


@pytest.mark.parametrize("kind", ["ssd", "ssd, wide state", "ssd, odd channels", "ssd, three lanes of states",
                                  "ssd, matrix form 64", "ssd, matrix form 128"])
def test_long_portions_run_in_chunks_and_leave_the_same_state(kind):
    """bfloat16: a portion of several hundred tokens is cut into chunks that run side by side, a short one is
    walked in one piece; a long portion beside a single token of another request, then the same tokens in short
    portions: the outputs agree with the plain implementation and the float32 states that the two ways leave agree
    to float32 rounding."""
    from qwen3_from_scratch_b200.kernels import ops
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    table = mixers()
    # a state of 48: four lanes of which the last holds nothing; channels and states in multiples of 8 and 16 (the
    # form with 16-byte loads)
    table["ssd, three lanes of states"] = ({"hidden_size": 40, "num_heads": 4, "vdim": 16, "state": 48, "groups": 2,
                                            "norm_groups": 2, "conv": 4, "norm_eps": 1e-5},)
    # heads of 64 channels with a state of 64 or 128: the chunks run as matrix products on the tensor cores
    table["ssd, matrix form 64"] = ({"hidden_size": 40, "num_heads": 4, "vdim": 64, "state": 64, "groups": 2,
                                     "norm_groups": 4, "conv": 4, "norm_eps": 1e-5},)
    table["ssd, matrix form 128"] = ({"hidden_size": 40, "num_heads": 2, "vdim": 64, "state": 128, "groups": 1,
                                      "norm_groups": 1, "conv": 3, "norm_eps": 1e-5},)
    params = table[kind][0]
    assert ops.ssd_matrix_form(params["vdim"], params["state"]) == ("matrix" in kind)
    bench = MixerBench(create_part("mixer", PartSpec("ssd", params), name="m"), "bfloat16", max_tokens=1024, pages=8, seed=13)
    g = torch.Generator().manual_seed(14)
    x_of = {"a": torch.randn(700, 40, generator=g).to(torch.bfloat16), "b": torch.randn(3, 40, generator=g).to(torch.bfloat16)}
    fn = _ssd(params)
    want = {r: fn(x.double(), bench.ref, None)[0] for r, x in x_of.items()}
    with plain.bfloat16_projections():  # what rounding alone does over 700 tokens: the bound is three times that
        rounded = fn(x_of["a"].double(), bench.ref, None)[0]
    tol = max(TOL["bfloat16"], 3 * float((rounded - want["a"]).abs().max()) / float(want["a"].abs().max()))
    call = lambda x, ctx: bench.part.forward(x.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    assert ops.ssd_chunked_pays(torch.bfloat16, 697) and not ops.ssd_chunked_pays(torch.bfloat16, 100)
    states = []
    for steps in ([[("b", 2)], [("a", 697), ("b", 1)], [("a", 3)]],
                  [[("b", 2)]] + [[("a", 100)]] * 3 + [[("a", 100), ("b", 1)]] + [[("a", 100)]] * 3):
        got = {r: [] for r in x_of}
        for step in steps:
            for r, y in bench.run(step, x_of, call).items():
                got[r].append(y)
        for r in x_of:
            close(torch.cat(got[r]), want[r], "bfloat16", f"{kind} {r}", tol=tol)
        slot = bench.manager.slot("a")
        states.append({k: t[slot].clone() for k, t in bench.storage.states.items()})
        bench.manager.close("a")
        bench.manager.close("b")
    for k in states[0]:
        scale = float(states[0][k].abs().max())
        assert float((states[0][k] - states[1][k]).abs().max()) <= 2e-5 * scale, k


@pytest.mark.parametrize("dtype", list(DT))
def test_sharp_attention_reads_keys_far_back_and_at_page_borders(dtype):
    """A scale so large that nearly every query gives all its weight to one key, which random weights put
    anywhere in the past: hundreds of tokens back, on a page's first or last slot, the very first token, the
    query's own.  A key that is lost or shifted by one changes that query's output entirely.  As a whole prompt,
    then in portions and single tokens."""
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    W, n, page = 32, 430, 16
    params = {"hidden_size": W, "num_heads": 4, "dim": 16, "rot_dim": 16, "vdim": 24, "kv_rank": 64, "q_rank": 32,
              "scale": 6.0, "norm_eps": 1e-5,
              "position": PartSpec("rotary_stretched", {"dims": 16, "base": 10000.0, "scaling": None})}
    part = create_part("mixer", PartSpec("latent_attention", params), name="m")
    bench = MixerBench(part, dtype, page_size=page, pages=64, max_tokens=512, seed=41)
    x = torch.randn(n, W, generator=torch.Generator().manual_seed(42)).to(DT[dtype])
    plain_fn = _latent(params)
    want = plain_fn(x.double(), bench.ref, None)[0]
    # what the plain scores say about where the weight goes
    m = {"heads": 4, "dim": 16, "rot_dim": 16, "kv_rank": 64}
    cq = plain.rms_norm(x.double() @ bench.ref["dq"].t(), bench.ref["dq.norm"], 1e-5)
    q = (cq @ bench.ref["uq"].t()).view(n, 4, 32)
    down = x.double() @ bench.ref["dkv"].t()
    c = plain.rms_norm(down[:, :64], bench.ref["dkv.norm"], 1e-5)
    freq, mag = plain.yarn_frequencies(16, 10000.0, None)
    pos = torch.arange(n)
    qr, kr = plain.rotate_half(q[..., 16:], pos, freq, mag), plain.rotate_half(down[:, None, 64:], pos, freq, mag)[:, 0]
    kp = (c @ bench.ref["uk"].t()).view(n, 4, 16)
    s = (torch.einsum("thd,nhd->htn", q[..., :16], kp) + torch.einsum("thd,nd->htn", qr, kr)) * 6.0
    s = s.masked_fill(~(pos[None, :] <= pos[:, None])[None], float("-inf"))
    top, arg = torch.softmax(s, -1).max(-1)  # [heads, n]
    sharp = top > 0.9
    back = (pos[None, :] - arg)[sharp]
    assert sharp.float().mean() > 0.5 and int((back > 100).sum()) > 50 and int((back == 0).sum()) > 0
    assert int((arg[sharp] % page == 0).sum()) > 5 and int((arg[sharp] % page == page - 1).sum()) > 5
    assert int((arg[sharp] == 0).sum()) > 0
    call = lambda rows, ctx: part.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    # bfloat16 rounds scores of this size by a few tenths, which moves a weight that is not yet saturated: there
    # only the queries all of whose heads give a key more than 0.99 are compared (every lost key still shows)
    rows = torch.arange(n) if dtype == "float32" else (top > 0.99).all(0).nonzero()[:, 0]
    assert rows.numel() > 80 and int(((pos[None, :] - arg)[:, rows] > 100).sum()) > 20
    got = bench.run([("r", n)], {"r": x}, call)["r"]
    close(got[rows], want[rows], dtype, "whole prompt")
    bench.manager.close("r")
    cuts = [47, 1, 1, 150, 1] + [2] * 40 + [17, 15, 33] + [1] * (n - 47 - 153 - 80 - 65)
    pieces = torch.cat([bench.run([("r", k)], {"r": x}, call)["r"] for k in cuts])
    close(pieces[rows], want[rows], dtype, "portions and single tokens")


@pytest.mark.parametrize("dtype", list(DT))
def test_a_slow_decay_carries_the_first_token_to_the_end(dtype):
    """Decays near one and no skip: what the first token wrote into the state is still most of the output
    hundreds of tokens later, through portions and single tokens and beside another request's tokens."""
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    params = {"hidden_size": 32, "num_heads": 4, "vdim": 8, "state": 16, "groups": 2, "norm_groups": 1, "conv": 3,
              "norm_eps": 1e-5}

    def tweak(dev, ref):
        for tensors, pre in ((dev, "m."), (ref, "")):
            tensors[pre + "A_log"].fill_(-7.0)     # exp(-exp(-7) step): a decay within a thousandth of one
            tensors[pre + "D"].fill_(0.0)
            tensors[pre + "conv.b"].fill_(0.0)     # a quiet input then writes next to nothing into the state

    part = create_part("mixer", PartSpec("ssd", params), name="m")
    bench = MixerBench(part, dtype, page_size=8, pages=8, max_tokens=512, seed=51, tweak=tweak)
    g = torch.Generator().manual_seed(52)
    n = 400
    x = 0.02 * torch.randn(n, 32, generator=g)
    x[0] = 3 * torch.randn(32, generator=g)
    x_of = {"r": x.to(DT[dtype]), "o": torch.randn(9, 32, generator=g).to(DT[dtype])}
    fn = _ssd(params)
    want = fn(x_of["r"].double(), bench.ref, None)[0]
    quiet = x_of["r"].clone()
    quiet[0] = 0
    assert float((want[-1] - fn(quiet.double(), bench.ref, None)[0][-1]).abs().max()) > 0.5 * float(want[-1].abs().max())
    call = lambda rows, ctx: part.forward(rows.cuda().contiguous(), ctx, 0, True)  # noqa: E731
    close(bench.run([("r", n)], x_of, call)["r"], want, dtype, "whole")
    bench.manager.close("r")
    got = []
    for step in ([("r", 1)], [("r", 2), ("o", 4)], [("r", 290)], [("o", 1), ("r", 1)], [("r", 2)], [("r", 64), ("o", 4)]) \
            + tuple([("r", 1)] for _ in range(40)):
        got.append(bench.run(list(step), x_of, call)["r"])
    close(torch.cat(got), want, dtype, "portions")


@pytest.mark.parametrize("dtype", list(DT))
def test_block_over_three_streams(dtype):
    """One block alone: what it leaves open is applied by hand, and the streams agree with the plain layer."""
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    W, S, T = 40, 3, 21
    norm = PartSpec("rms_norm", {"dim": W, "eps": 1e-5, "suffix": ""})
    params, _ = mixers()["ssd"]
    spec = PartSpec("hyper_pre_norm", {
        "norm1": norm, "mixer": PartSpec("ssd", params), "norm2": norm, "streams": S, "width": W,
        "feed_forward": PartSpec("dense_mlp", {"hidden_size": W, "intermediate_size": 56, "activation": "gelu_tanh",
                                               "names": {"up": "up", "down": "down"}}),
        "names": {"mixer": "mix", "feed_forward": "mlp"}})
    block = create_part("block", spec, name="l0")
    bench = MixerBench(block, dtype, seed=61)
    for k in ("hc1.mix", "hc2.mix"):  # near the identity, like a model's
        bench.dev["l0." + k].copy_(torch.eye(S) + 0.5 * bench.ref[k].float())
        bench.ref[k] = bench.dev["l0." + k].double().cpu()
    xs = torch.randn(T, S, W, generator=torch.Generator().manual_seed(62))
    config = {"layers": [{"type": "mamba2", "mixer": {"heads": 6, "vdim": 8, "state": 24, "groups": 3, "norm_groups": 2},
                          "mlp": {"kind": "dense", "ff": 56}}], "norm": {"eps": 1e-5}}
    w = {"l0." + k: v for k, v in bench.ref.items()}
    want, _ = plain.layer(xs.double().transpose(0, 1), w, config, 0, None)

    def call(_, ctx):
        streams = xs.cuda().contiguous()
        pending = block.forward(streams, None, ctx, 0, True)
        return torch.einsum("ft,xfw->xtw", pending.mix, streams) + pending.write[None, :, None] * pending.delta.float()[:, None, :]

    got = bench.run([("a", T)], {"a": torch.zeros(T, 1)}, call)["a"]
    close(got.transpose(0, 1), want, dtype, "streams after the block")


# ---------------------------------------------------------------------- the tensor-core kernel against the plain one
@pytest.mark.parametrize("H,rank,rot,page", [(16, 128, 64, 16), (5, 64, 32, 4), (17, 64, 64, 8), (16, 512, 64, 16),
                                             (40, 256, 32, 16), (1, 128, 8, 32)])
def test_tensor_core_latent_attention_equals_the_plain_kernel(H, rank, rot, page):
    """bfloat16: a batch of a long portion, a portion that ends exactly on a tile's edge, a short one and two single
    tokens, scattered over pages in another order than the tokens'; then single tokens alone with their keys cut
    into ranges that are merged."""
    from types import SimpleNamespace
    from qwen3_from_scratch_b200.kernels import ops
    assert ops.latent_attention_fast(torch.bfloat16, rank, rot)
    g = torch.Generator().manual_seed(H * 1000 + rank)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731

    def batch(q_lens, kv_lens):
        B, T = len(q_lens), sum(q_lens)
        need = [-(-n // page) for n in kv_lens]
        pages = sum(need) + 3
        order = torch.randperm(pages, generator=g).tolist()
        table = torch.full((B, max(need) + 1), -1, dtype=torch.int32)
        at = 0
        for b, n in enumerate(need):
            table[b, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
            at += n
        c_pages = torch.randn(pages, 1, page, rank, generator=g).to(torch.bfloat16).cuda()
        r_pages = torch.randn(pages, 1, page, rot, generator=g).to(torch.bfloat16).cuda()
        q_abs = (torch.randn(H, T, rank, generator=g) * 0.5).cuda()
        q_rot = (torch.randn(T, H, rot, generator=g) * 0.5).to(torch.bfloat16).cuda()
        starts = [0] + torch.tensor(q_lens).cumsum(0).tolist()
        ctx = SimpleNamespace(
            positions=i32([kv_lens[b] - q_lens[b] + i for b in range(B) for i in range(q_lens[b])]),
            tok_seq=i32([b for b in range(B) for _ in range(q_lens[b])]), q_start=i32(starts), kv_len=i32(kv_lens),
            num_seqs=B, max_q_len=max(q_lens), max_kv_len=max(kv_lens))
        return q_abs, q_rot, c_pages, r_pages, ctx, table.cuda(), T

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = (rank + rot) ** -0.5
    for q_lens, kv_lens, scratch in (([70, 32, 3, 1, 1], [200, 64, 3, 77, 1], False), ([1, 1, 1], [300, 1, 33], True),
                                     ([1], [1500], True)):
        q_abs, q_rot, c_pages, r_pages, ctx, table, T = batch(q_lens, kv_lens)
        want = torch.empty(T, H * rank, dtype=torch.bfloat16, device="cuda")
        ops.latent_attention(q_abs, q_rot, c_pages, r_pages, ctx, table, want, scale, status, kernel="plain")
        got = torch.full_like(want, float("nan"))
        partial = torch.empty(ops.latent_partial_numel(len(q_lens), H, rank), device="cuda") if scratch else None
        if scratch and max(kv_lens) > 1000:
            assert ops.latent_decode_splits(len(q_lens), H, max(kv_lens)) > 1
        ops.latent_attention(q_abs, q_rot, c_pages, r_pages, ctx, table, got, scale, status, partial=partial, kernel="mma")
        assert int(status.item()) == 0
        # the tensor-core kernel rounds the absorbed query and each weight to bfloat16; both round the output once
        scale_of = float(want.float().abs().max())
        assert float((got.float() - want.float()).abs().max()) <= 1.5e-2 * scale_of, (q_lens, kv_lens)


# ---------------------------------------------------------------------- whole models
def tolerance(dtype, cfg, w, seqs):
    """float32: the harness's bound.  bfloat16: three times what rounding alone does to these prompts in the plain
    implementation (projections' operands and results rounded to bfloat16), and no less than the harness's bound."""
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
@pytest.mark.parametrize("key", ["x", "z"])
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
    """bfloat16 at the serving kernels' sizes with pages of 16: a prompt of 700 tokens whole and cut into long and
    short portions with single tokens between them."""
    cfg, w = plain.read_model_folder(folders["z"])
    ids = tokens(cfg["vocab"], 700, 77)
    want = {"a": plain.forward_logits(cfg, w, ids)}
    tol = tolerance("bfloat16", cfg, w, {"a": ids})
    for name, cuts in (("whole", [700]), ("portions", [300, 1, 250, 1, 1, 130, 17])):
        got = replay(folders["z"], "bfloat16", {"a": ids}, lambda r, cuts=cuts: [r.step([("a", n)]) for n in cuts],
                     page_size=16, num_pages=64, max_seqs=2, max_step_tokens=1024)
        assert_close(got, want, "bfloat16", f"z long {name}", tol=tol)


def test_long_decoding_through_graphs(folders):
    """300 single tokens after a short prompt, replayed from CUDA graphs: states and latents are carried on the
    device from step to step; the last logits still agree with the plain implementation in float32."""
    cfg, w = plain.read_model_folder(folders["y"])
    ids = tokens(cfg["vocab"], 310, 71)
    want = {"a": plain.forward_logits(cfg, w, ids)}

    def schedule(r):
        r.step([("a", 10)])
        for _ in range(300):
            r.step([("a", 1)])

    got = replay(folders["y"], "float32", {"a": ids}, schedule, num_pages=64, max_seqs=2)
    assert_close(got, want, "float32", "long decoding")


def test_float32_cuts_give_identical_bits(folders):
    """In float32 every sum has an order that depends only on the token, so a prompt whole, in portions and
    token by token gives the same bits."""
    cfg, _ = plain.read_model_folder(folders["x"])
    ids = tokens(cfg["vocab"], 45, 81)
    runs = [replay(folders["x"], "float32", {"a": ids}, s)["a"] for s in (
        lambda r: r.step([("a", 45)]),
        lambda r: [r.step([("a", n)]) for n in (7, 2, 1, 20, 15)],
        lambda r: [r.step([("a", 1)]) for _ in range(45)])]
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[0], runs[2])


# ---------------------------------------------------------------------- the engine's entry points
@pytest.mark.parametrize("key", ["x", "y"])
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
    cfg, _ = plain.read_model_folder(folders["x"])
    prompts = [tokens(cfg["vocab"], n, 90 + i) for i, n in enumerate([30, 28, 26])]
    alone = SyncEngine(folders["x"], dtype="float32", block_size=4, num_pages=64, max_num_seqs=4, max_num_tokens=64)
    want = [alone.generate(p, max_new_tokens=24, ignore_eos=True) for p in prompts]
    tight = SyncEngine(folders["x"], dtype="float32", block_size=4, num_pages=34, max_num_seqs=4, max_num_tokens=64)
    results, _ = tight.batch_generate(prompts, max_new_tokens=24, ignore_eos=True)
    assert [r.token_ids for r in results] == want
    assert tight.scheduler.num_preemptions > 0


@pytest.mark.parametrize("dtype", list(DT))
def test_trace_replay_program_and_command_line(folders, tmp_path, dtype):
    folder = folders["x"]
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
