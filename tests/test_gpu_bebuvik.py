"""The Bebuvik design on the GPU against the plain implementation (tests/plain/plain_bebuvik.py): every
mechanism alone, then whole models replayed whole, token by token, in portions down to two tokens and mixed
with other requests on a pool so small that pages and slots are used again; generation through the scheduler.

Where random weights would hide a fault the inputs are made so that it shows: one key far back whose score
stands out, queries just inside and just outside a window, sinks that take most of a row's weight."""

import json
import math
import subprocess
import sys

import numpy as np
import pytest
import torch

from bebuvik_tools import CONFIGS, PAGE_SIZES, make, plain_rows
from helpers import random_tokens
from plain import plain_bebuvik as plain
from trace_tools import ROOT, mixed_trace, portions_trace, round64, run_trace_cli, run_trace_engine, tail_trace, whole_trace, worst_diff

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# |engine - plain float64| on logits that the soft cap keeps within a few units. float32: order of sums and the
# device's exp, tanh, sin, cos. bfloat16: three times the worst error measured per configuration.
TOL_F32 = 4e-5
TOL_BF16_MEASURED = {"P": 0.057, "Q": 0.136, "R": 0.035, "S": 0.081, "T": 0.105}
LENGTHS = {"P": [70, 45, 100, 33, 2, 64, 17, 1], "Q": [130, 64, 97, 33, 150, 5], "R": [50, 33, 80, 17, 64],
           "S": [90, 41, 120, 8, 64, 33], "T": [60, 100, 31, 64, 9, 70]}


def tol(name, dtype):
    return TOL_F32 if dtype == "float32" else 3.0 * TOL_BF16_MEASURED[name]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("bebuvik")
    return {name: make(root / name, name) for name in CONFIGS}


def _requests(name):
    v = CONFIGS[name]["vocab"]
    return {f"{name}{i}": random_tokens(n, v, seed=31 * i + n) for i, n in enumerate(LENGTHS[name])}


_expected = {}


def _expect(models, name):
    if name not in _expected:
        _, cfg, w = models[name]
        _expected[name] = plain_rows(cfg, w, _requests(name))
    return _expected[name]


# ---------------------------------------------------------------- mechanisms alone


def _state_batch(lengths, starts, slots):
    """The step arrays a kernel reads, for entries of the given lengths."""
    q_start = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    token_req = np.concatenate([np.full(n, i) for i, n in enumerate(lengths)]).astype(np.int32)
    positions = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lengths)]).astype(np.int32)
    f = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)
    return f(q_start), f(token_req), f(positions), f(starts), f(slots)


def test_bigram_embedding_carries_the_previous_token_across_steps_and_slots():
    from quantinfer_b200 import kernels

    torch.manual_seed(0)
    V, Hd, B = 57, 24, 13
    table, big = torch.randn(V, Hd), torch.randn(B + 1, Hd)
    seqs = {0: random_tokens(23, V, 1), 2: random_tokens(9, V, 2), 1: random_tokens(14, V, 3)}
    want = {s: plain.embed(t, table, big, {"buckets": B, "mul_prev": 11, "mul_cur": 3}) for s, t in seqs.items()}
    state = torch.full((4, 1), 12345, dtype=torch.int32, device=DEV)      # a slot's old owner left something behind
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    done = {s: 0 for s in seqs}
    cuts = [(0, 5), (2, 1), (1, 2), (0, 1), (2, 8), (1, 12), (0, 17)]
    for step in range(0, len(cuts), 2):
        group = cuts[step:step + 2]
        lengths = [n for _, n in group]
        starts = [done[s] for s, _ in group]
        ids = sum([seqs[s][done[s]:done[s] + n] for s, n in group], [])
        q_start, token_req, positions, _, slots = _state_batch(lengths, starts, [s for s, _ in group])
        out = torch.empty((len(ids), Hd), device=DEV)
        kernels.embedding_bigram(table.to(DEV), big.to(DEV), torch.tensor(ids, dtype=torch.int32, device=DEV), positions,
                                 token_req, q_start, slots, state, out, B, 11, 3, status)
        a = 0
        for s, n in group:
            assert torch.equal(out[a:a + n].cpu(), want[s][done[s]:done[s] + n]), (s, done[s])
            a += n
            done[s] += n
    assert int(status.item()) == 0 and done == {s: len(t) for s, t in seqs.items()}


@pytest.mark.parametrize("taps", [1, 2, 4, 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_short_conv_in_portions_of_every_size(taps, dtype):
    """Two filters over one input, three requests in one launch, cut into portions of one to many tokens so that a
    portion is shorter than, equal to and longer than the filter; slots used in another order than the entries."""
    from quantinfer_b200 import kernels

    torch.manual_seed(taps)
    ch = 37
    w = torch.randn(2, ch, taps)
    seqs = {3: torch.randn(29, ch), 0: torch.randn(11, ch), 1: torch.randn(17, ch)}
    want = {s: [x + plain.causal_conv(x, w[k]) for k in range(2)] for s, x in seqs.items()}
    state = torch.full((4, max(taps - 1, 1), ch), 7.0, device=DEV)[:, :taps - 1]   # stale values of an earlier owner
    state = state.contiguous()
    wd = w.permute(0, 2, 1).contiguous().to(DEV)
    plans = {3: [1, 1, 2, 3, 1, 4, 5, 2, 10], 0: [3, 1, 1, 6], 1: [17]}
    done = {s: 0 for s in seqs}
    while any(plans.values()):
        group = [(s, plans[s].pop(0)) for s in (1, 3, 0) if plans[s]]
        lengths, starts = [n for _, n in group], [done[s] for s, _ in group]
        h = torch.cat([seqs[s][done[s]:done[s] + n] for s, n in group]).to(DEV)
        q_start, token_req, _, start_pos, slots = _state_batch(lengths, starts, [s for s, _ in group])
        outs = [torch.empty(h.shape, dtype=dtype, device=DEV) for _ in range(2)]
        copy = torch.empty(h.shape, dtype=dtype, device=DEV)
        kernels.short_conv(h, wd, state if taps > 1 else None, outs, copy, token_req, q_start, start_pos, slots)
        a = 0
        for s, n in group:
            for k in range(2):
                ref = want[s][k][done[s]:done[s] + n]
                err = float((outs[k][a:a + n].float().cpu() - ref).abs().max())
                assert err < (1e-5 if dtype == torch.float32 else 0.05), (s, done[s], n, k, err)
            assert torch.equal(copy[a:a + n].cpu(), seqs[s][done[s]:done[s] + n].to(dtype))
            a += n
            done[s] += n


@pytest.mark.parametrize("taps", [1, 3, 4])
@pytest.mark.parametrize("in_dtype, dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16)])
def test_short_conv_with_four_channels_a_thread(taps, in_dtype, dtype):
    """A step of 256 rows and more, with a channel count that is a multiple of four, takes the form with 16-byte
    accesses; the same rows in steps of fewer take the form with a thread a channel. Both must give the same bits, and
    the formula's values: three requests in one launch (one continues a sequence whose state an earlier step left, one
    is a single token, one starts at zero over a stale slot), two filters, a copy of the input."""
    from quantinfer_b200 import kernels

    torch.manual_seed(taps + 10)
    ch = 40
    w = torch.randn(2, ch, taps)
    wd = w.permute(0, 2, 1).contiguous().to(DEV)
    seqs = {2: torch.randn(30 + 200, ch).to(in_dtype).float(), 0: torch.randn(5 + 1, ch).to(in_dtype).float(), 1: torch.randn(90, ch).to(in_dtype).float()}
    want = {s: [x + plain.causal_conv(x, w[k]) for k in range(2)] for s, x in seqs.items()}
    results = []
    for big in (True, False):
        state = torch.full((3, max(taps - 1, 1), ch), 7.0, device=DEV)[:, :taps - 1].contiguous()
        got = {s: [[], []] for s in seqs}
        # first the beginnings of requests 2 and 0 (their state stays behind), then the step of 291 rows, whole or in pieces
        plan = [[(2, 0, 30), (0, 0, 5)]] + ([[(2, 30, 200), (0, 5, 1), (1, 0, 90)]] if big else
                                            [[(2, 30, 100), (0, 5, 1), (1, 0, 50)], [(2, 130, 100), (1, 50, 40)]])
        for group in plan:
            lengths, starts = [n for _, _, n in group], [a for _, a, _ in group]
            h = torch.cat([seqs[s][a:a + n] for s, a, n in group]).to(in_dtype).to(DEV)
            q_start, token_req, _, start_pos, slots = _state_batch(lengths, starts, [s for s, _, _ in group])
            outs = [torch.empty(h.shape, dtype=dtype, device=DEV) for _ in range(2)]
            copy = torch.empty(h.shape, dtype=dtype, device=DEV)
            kernels.short_conv(h, wd, state if taps > 1 else None, outs, copy, token_req, q_start, start_pos, slots)
            assert torch.equal(copy.float().cpu(), h.float().cpu().to(dtype).float())
            at = 0
            for s, a, n in group:
                for k in range(2):
                    got[s][k].append(outs[k][at:at + n].float().cpu())
                at += n
        results.append({s: [torch.cat(g) for g in gs] for s, gs in got.items()})
    for s in seqs:
        for k in range(2):
            assert torch.equal(results[0][s][k], results[1][s][k]), (s, k)
            err = float((results[0][s][k] - want[s][k]).abs().max())
            assert err < (2e-5 if dtype == torch.float32 else 0.06), (s, k, err)


def test_small_kernels_against_their_formulas():
    from quantinfer_b200 import kernels

    torch.manual_seed(5)
    n, ch = 7, 53
    for dt in (torch.float32, torch.bfloat16):
        g, y0, y1 = (torch.randn(n, 2 * ch) * 2).to(dt), torch.randn(n, ch).to(dt), torch.randn(n, ch).to(dt)
        b0, b1 = torch.randn(ch), torch.randn(ch)
        out = torch.empty((n, ch), device=DEV)
        kernels.gated_sum(g.to(DEV), b0.to(DEV), b1.to(DEV), y0.to(DEV), y1.to(DEV), out)
        ref = torch.sigmoid(g.float()[:, :ch] + b0) * y0.float() + torch.sigmoid(g.float()[:, ch:] + b1) * y1.float()
        assert float((out.cpu() - ref).abs().max()) < 2e-6
        kernels.gated_sum(g[:, :ch].contiguous().to(DEV), b0.to(DEV), None, y0.to(DEV), None, out)
        assert float((out.cpu() - torch.sigmoid(g.float()[:, :ch] + b0) * y0.float()).abs().max()) < 2e-6
        x = (torch.randn(n, ch) * 3).to(dt)
        act = torch.empty_like(x, device=DEV)
        kernels.activation(x.to(DEV), act, "gelu_tanh")
        assert float((act.float().cpu() - plain.gelu_tanh(x.float())).abs().max()) < (2e-6 if dt == torch.float32 else 2e-2)
    z = torch.randn(5, 33) * 40
    zd = z.to(DEV)
    kernels.softcap(zd, 11.0)
    assert float((zd.cpu() - 11.0 * torch.tanh(z / 11.0)).abs().max()) < 5e-6
    # per-head products from rows that hold more than the heads, into rows that hold more too
    heads, xw, k, N, ow = 3, 11, 6, 5, 9
    x, w = torch.randn(n, heads * xw + 4), torch.randn(heads, N, k)
    out = torch.zeros(n, heads * ow, device=DEV)
    kernels.head_linear(x.to(DEV), xw, 2, k, w.to(DEV), out, ow, 3)
    for h in range(heads):
        ref = x[:, h * xw + 2:h * xw + 2 + k] @ w[h].t()
        assert float((out.cpu()[:, h * ow + 3:h * ow + 3 + N] - ref).abs().max()) < 1e-5
        assert float(out.cpu()[:, h * ow:h * ow + 3].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scalar_norm_and_dense_feed_forward_parts(dtype):
    from quantinfer_b200.config import DenseFeedForwardSpec, NormSpec
    from quantinfer_b200.parts import Runtime, build_part

    torch.manual_seed(2)
    rt = Runtime(dtype, DEV)
    norm = build_part("norm", NormSpec(52, 2e-5, "n", "rmsnorm_scalar"), rt)
    assert {k: v.shape for k, v in norm.tensor_needs().items()} == {"n": ()}
    norm.load({"n": torch.tensor(1.3)})
    resid, delta = torch.randn(6, 52), torch.randn(6, 52)
    out = norm.forward(resid.to(DEV), delta.to(DEV))
    ref = plain.scalar_norm(resid + delta, torch.tensor(1.3), 2e-5)
    assert float((out.float().cpu() - ref).abs().max()) < (1e-5 if dtype == torch.float32 else 3e-2)
    ff = build_part("ffn", DenseFeedForwardSpec(52, 70, "gelu_tanh", "f."), rt)
    w = {"f.up": (torch.randn(70, 52) / 7).to(dtype), "f.down": (torch.randn(52, 70) / 8).to(dtype)}
    ff.load(w)
    x = torch.randn(6, 52).to(dtype)
    y = ff.forward(x.to(DEV))
    ref = plain.dense_ff(x.float(), w["f.up"].float(), w["f.down"].float())
    assert float((y.float().cpu() - ref).abs().max()) < (2e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("R, r, H, window, page", [(64, 16, 5, 37, 64), (32, 16, 1, None, 8), (128, 64, 8, 17, 16),
                                                    (64, 32, 70, 33, 32), (256, 64, 3, 100, 16), (32, 32, 64, 1, 8)])
def test_tensor_core_latent_attention_against_float64(R, r, H, window, page):
    """The flash kernel alone on a batch of three decode tokens in front of portions of 2, 130 and 37 tokens that
    start in the middle of pages, over shuffled pages; one far key of the long request is made to dominate; the
    pages before every window hold NaN (they may be free again and must not be read into the sums)."""
    from quantinfer_b200 import kernels

    torch.manual_seed(R + r + H)
    W = R + r
    lengths, starts = [1, 1, 1, 2, 130, 37], [0, 63, 200, 14, 9, 250]
    n_req, max_blocks = len(lengths), 48
    num_pages = sum(-(-(s + n) // page) for s, n in zip(starts, lengths)) + 3
    order = torch.randperm(num_pages).tolist()
    table = torch.full((n_req, max_blocks), -1, dtype=torch.int32)
    cache = torch.full((num_pages, page, W), float("nan"), dtype=torch.bfloat16)
    rows = []
    for e, (s, n) in enumerate(zip(starts, lengths)):
        kv = (torch.randn(s + n, W) * 0.7).to(torch.bfloat16)
        if e == 4:
            kv[20, R:] *= 6.0            # a far key whose rotated part stands out
        lo = 0 if window is None else max(0, s - window + 1)
        for b in range(lo // page, -(-(s + n) // page)):
            pg = order.pop()
            table[e, b] = pg
            seg = kv[b * page:(b + 1) * page]
            cache[pg, :seg.shape[0]] = seg
            if b * page < lo:
                cache[pg, :lo - b * page] = float("nan")      # before the first query's window: never to be used
        rows.append(kv)
    n = sum(lengths)
    q = (torch.randn(n, H, W) * 0.7).to(torch.bfloat16)
    sink = torch.randn(H)
    scale = 1.0 / math.sqrt(W)
    ref = torch.zeros(n, H, R, dtype=torch.float64)
    t = 0
    for e, (s, ln) in enumerate(zip(starts, lengths)):
        for i in range(ln):
            p = s + i
            lo = 0 if window is None else max(0, p - window + 1)
            kv = rows[e][lo:p + 1].double()
            sc = torch.einsum("hw,jw->hj", q[t].double(), kv) * scale
            mx = torch.maximum(sc.max(dim=1).values, sink.double())
            ex = torch.exp(sc - mx[:, None])
            ref[t] = (ex / (ex.sum(dim=1) + torch.exp(sink.double() - mx))[:, None]) @ kv[:, :R]
            t += 1
    q_start, token_req, positions, start_pos, _ = _state_batch(lengths, starts, list(range(n_req)))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = {}
    for impl, ranges in (("mma", 1), ("generic", 1), ("mma", 3), ("mma", 16)):       # 16: more key ranges than some rows have tiles
        out = torch.full((n, H, R), 7.0, dtype=torch.bfloat16, device=DEV)
        kernels.latent_attention(q.to(DEV), out, cache.to(DEV), sink.to(DEV), table.to(DEV), q_start, start_pos, positions,
                                 token_req, scale, window or 0, status, impl=impl, key_ranges=ranges)
        outs[impl] = out.float().cpu().double()
        err = (outs[impl] - ref).abs().amax(dim=(1, 2))
        assert float(err.max()) < 0.03, (impl, ranges, int(err.argmax()), float(err.max()))
    assert int(status.item()) == 0
    table[4, (starts[4] + 60) // page] = -1                  # a page the long portion needs is missing: flagged, not read
    out = torch.empty((n, H, R), dtype=torch.bfloat16, device=DEV)
    kernels.latent_attention(q.to(DEV), out, cache.to(DEV), sink.to(DEV), table.to(DEV), q_start, start_pos, positions, token_req,
                             scale, window or 0, status, impl="mma")
    assert int(status.item()) == kernels.STATUS_BAD_PAGE


@pytest.mark.parametrize("n, heads, k, N", [(5, 6, 64, 64), (200, 3, 32, 80), (64, 70, 128, 16), (1, 2, 8, 8)])
def test_tensor_core_head_products_against_float64(n, heads, k, N):
    from quantinfer_b200 import kernels

    torch.manual_seed(n)
    xw, ow = k + 16, N + 8
    x, w = torch.randn(n, heads * xw + 8).to(torch.bfloat16), (torch.randn(heads, N, k) / math.sqrt(k)).to(torch.bfloat16)
    out = torch.zeros(n, heads * ow, dtype=torch.bfloat16, device=DEV)
    before = kernels.launches
    kernels.head_linear(x.to(DEV), xw, 8, k, w.to(DEV), out, ow, 2)
    assert kernels.launches == before + 1
    for h in range(heads):
        ref = x[:, h * xw + 8:h * xw + 8 + k].double() @ w[h].double().t()
        got = out.cpu()[:, h * ow + 2:h * ow + 2 + N].double()
        assert float((got - ref).abs().max()) < 0.02 * max(1.0, float(ref.abs().max())), h
        assert float(out.cpu()[:, h * ow:h * ow + 2].abs().max()) == 0.0


# ---------------------------------------------------------------- the mixer alone, with inputs made to show faults


def _mixer_engine(tmp_path, mixer, width, dtype, page_size, shared=False):
    """An engine of one or two layers whose LAST layer's mixer is the one under test (with `shared`, it reads
    the first layer's latent)."""
    from quantinfer_b200.engine import Engine
    from bebuvik_tools import draw_weights, write_folder

    layers = [{"type": "latent_attention", "mixer": dict(mixer), "mlp": None}]
    if shared:
        first = dict(mixer)
        layers = [{"type": "latent_attention", "mixer": first, "mlp": None},
                  {"type": "latent_attention", "mixer": dict(mixer, kv_from=0), "mlp": None}]
    cfg = {"architecture": "Bebuvik", "vocab": 16, "width": width, "norm": {"eps": 1e-6}, "layers": layers}
    w = draw_weights(cfg, 77)
    folder = write_folder(tmp_path / f"m{len(layers)}{dtype}", cfg, w)
    return Engine.from_folder(folder, dtype=dtype, page_size=page_size, max_tokens=512, max_requests=4, use_graphs=False), cfg, w


def _run_mixer(eng, layer, inputs, cuts, write_first=None):
    """Feeds `inputs` [T, width] through layer `layer`'s mixer in portions `cuts` for one request; with
    `write_first`, layer 0's mixer runs on those inputs first in every step (it fills the shared cache)."""
    from quantinfer_b200.engine import StepEntry

    eng.open("r")
    outs, a = [], 0
    for n in cuts:
        eng.cache.prepare("r", n)
        batch = eng.make_batch([StepEntry("r", [0] * n, [])])
        if write_first is not None:
            eng.model.blocks[0].mixer.forward(write_first[a:a + n].to(DEV, eng.dtype), batch, eng._views[0])
        y = eng.model.blocks[layer].mixer.forward(inputs[a:a + n].to(DEV, eng.dtype), batch, eng._views[layer])
        outs.append(y.float().cpu())
        eng.raise_on_status()
        eng.cache.commit("r")
        a += n
    eng.close("r")
    return torch.cat(outs)


CUTS = {"whole": lambda T: [T], "one by one": lambda T: [1] * T,
        "portions": lambda T: _cycle(T, (2, 7, 3, 16, 2, 5, 31, 1)), "prompt then decode": lambda T: [T - 20] + [1] * 20}


def _cycle(T, sizes):
    out, i = [], 0
    while sum(out) < T:
        out.append(min(sizes[i % len(sizes)], T - sum(out)))
        i += 1
    return out


@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("window", [None, 9, 16, 17])
def test_a_far_key_and_the_windows_edges_show_in_the_mixer(tmp_path, cut, window):
    """One position's input is scaled so that its rotated key part gives it by far the largest score for every
    later query that sees it. Without a window every later row is then dominated by that one value; with a
    window the rows up to `window - 1` places later are, and the row `window` places later is not: a window that
    is one off, a key lost at a page's border or a stale page changes those rows by far more than the bound."""
    mixer = {"heads": 3, "dim": 8, "rot_dim": 8, "vdim": 10, "kv_rank": 12, "rot": {"base": 100.0, "dims": 8}, "scale": 0.3}
    if window is not None:
        mixer["mask"] = {"size": window}
    eng, cfg, w = _mixer_engine(tmp_path, mixer, 24, "float32", page_size=8)
    T, far = 75, 23                      # position 23: the last row of a page of eight
    torch.manual_seed(3)
    x = torch.randn(T, 24) * 0.3
    x[far] *= 40.0                       # the latent is normalised, the rotated key part is not
    ref, _ = plain.latent_attention(x.double(), {k: v.double() for k, v in w.items()}, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6,
                                    list(range(T)), None)
    got = _run_mixer(eng, 0, x, CUTS[cut](T))
    err = (got.double() - ref).abs().max(dim=1).values
    assert float(err.max()) < 2e-4, (int(err.argmax()), float(err.max()))
    # the test's premise: the far key matters where it is seen and the rows differ across the window's edge
    if window is not None:
        inside, outside = far + window - 1, far + window
        assert float((ref[inside] - ref[outside]).abs().max()) > 50 * 2e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sinks_take_their_share_and_a_reader_uses_its_own_weights_on_a_shared_latent(tmp_path, dtype):
    """A layer that reads another layer's cache: same latent, own queries, key and value expansion, window and
    sinks. Large sinks shrink every row; a sink left out, scaled or counted twice shows at once."""
    mixer = {"heads": 4, "dim": 16, "rot_dim": 16, "vdim": 16, "kv_rank": 32, "rot": {"base": 10000.0, "dims": 16}, "scale": 0.18,
             "mask": {"size": 20}}
    eng, cfg, w = _mixer_engine(tmp_path, mixer, 32, dtype, page_size=16, shared=True)
    w = dict(w)
    w["l1.mix.sink"] = torch.tensor([4.0, -3.0, 0.0, 9.0], dtype=torch.bfloat16)
    eng.model.blocks[1].mixer.sink = w["l1.mix.sink"].float().to(DEV)
    T = 50
    torch.manual_seed(4)
    x0, x1 = torch.randn(T, 32).to(torch.bfloat16).float(), torch.randn(T, 32).to(torch.bfloat16).float()
    wd = {k: v.double() for k, v in w.items()}
    _, latent = plain.latent_attention(x0.double(), wd, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6, list(range(T)), None)
    ref, _ = plain.latent_attention(x1.double(), wd, "l1.mix.", cfg["layers"][1]["mixer"], 1e-6, list(range(T)), latent)
    no_sink = dict(wd)
    no_sink["l1.mix.sink"] = torch.full((4,), -1e9, dtype=torch.float64)
    bare, _ = plain.latent_attention(x1.double(), no_sink, "l1.mix.", cfg["layers"][1]["mixer"], 1e-6, list(range(T)), latent)
    assert float((bare - ref).abs().max()) > 0.3              # the sinks matter in this test
    for cut in ("whole", "portions", "one by one"):
        got = _run_mixer(eng, 1, x1, CUTS[cut](T), write_first=x0)
        err = float((got.double() - ref).abs().max())
        assert err < (2e-4 if dtype == "float32" else 6e-2), (cut, err)


# ---------------------------------------------------------------- whole models, replayed


def _family(name, reqs, family):
    longest = round64(max(LENGTHS[name]))
    if family == "whole":
        return whole_trace(reqs), longest
    if family == "tail":
        return tail_trace(reqs, 48), longest
    if family == "portions":
        return portions_trace(reqs), longest
    steps, peak = mixed_trace(reqs, seed=5, max_live=4, max_tokens=longest + 2 * 64)
    assert sum(round64(n) for n in LENGTHS[name]) > peak and max(len(s["entries"]) for s in steps) >= 3
    return steps, peak


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_replay_family(models, name, dtype, family):
    folder, cfg, w = models[name]
    steps, max_tokens = _family(name, _requests(name), family)
    got = run_trace_engine(folder, dtype, steps, max_tokens, PAGE_SIZES[name])
    worst, where = worst_diff(got, _expect(models, name))
    print(f"measured {name} {dtype} {family}: {worst:.3g} at {where}")
    assert worst <= tol(name, dtype), f"first/worst difference {worst} at (request, position) {where}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(models, dtype):
    """bin/trace_run as a child process, the default page size, a mixed trace in which pages and slots are used again."""
    folder, cfg, w = models["Q"]
    reqs = _requests("Q")
    steps, peak = mixed_trace(reqs, seed=9, max_live=4, max_tokens=round64(max(LENGTHS["Q"])) + 128)
    got = _run_cli(folder, dtype, steps, peak, cfg["vocab"])
    worst, where = worst_diff(got, _expect(models, "Q"))
    assert worst <= tol("Q", dtype), (worst, where)


def _run_cli(folder, dtype, steps, max_tokens, vocab):
    import tempfile
    from pathlib import Path

    from trace_tools import collect

    with tempfile.TemporaryDirectory() as out:
        cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", out,
               "--max-tokens", str(max_tokens)]
        r = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-3000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
        outputs = {}
        for s in steps:
            wanted = sum(len(e["want"]) for e in s["entries"])
            if wanted:
                outputs[s["step"]] = np.fromfile(Path(out) / f"{s['step']}.f32", dtype="<f4").reshape(wanted, vocab)
    return collect(steps, outputs)


# ---------------------------------------------------------------- generation through the scheduler


def _plain_greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(plain.forward(cfg, w, toks, torch.float64)[-1].argmax()))
    return toks[len(prompt):]


@pytest.mark.parametrize("name, run_ahead, graphs", [("P", True, True), ("S", False, True), ("Q", True, False), ("T", True, True)])
def test_greedy_generation_through_the_scheduler(models, name, run_ahead, graphs):
    """Three prompts of unequal length taken in portions of five tokens while earlier ones already decode, decode
    steps replayed from CUDA graphs and launched ahead of the host: the plain implementation's tokens."""
    import quantinfer_b200 as q
    from quantinfer_b200.engine import Engine

    folder, cfg, w = models[name]
    prompts = [random_tokens(n, cfg["vocab"], seed=n) for n in (13, 1, 27)]
    eng = Engine.from_folder(folder, dtype="float32", page_size=PAGE_SIZES[name], max_tokens=512, max_requests=4, use_graphs=graphs)
    model = q.Model.from_engine(eng, max_batch_tokens=16, chunk_size=5, run_ahead=run_ahead)
    got = model.generate_batch(prompts, max_new_tokens=10, eos_token_id=None)
    for p, g in zip(prompts, got):
        assert g == _plain_greedy(cfg, w, p, 10), (name, len(p))
    # again on the same engine: slots and pages of the first call are used again, state must start afresh
    assert model.generate_batch(prompts[::-1], max_new_tokens=10, eos_token_id=None) == got[::-1]
    assert model.generate_tokens(prompts[2], max_new_tokens=10, eos_token_id=None) == got[2]


def test_command_line_generates_the_same_tokens(models):
    folder, cfg, w = models["R"]
    prompt = random_tokens(9, cfg["vocab"], seed=1)
    r = subprocess.run([sys.executable, str(ROOT / "bin" / "quantinfer"), "generate", "--input", str(folder), "--tokens",
                        ",".join(map(str, prompt)), "--max-new-tokens", "10", "--dtype", "float32", "--page-size", "16"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("generated_tokens=")][0]
    assert json.loads(line.split("=", 1)[1]) == _plain_greedy(cfg, w, prompt, 10)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_windows_and_pages(models, dtype):
    """Three tokens of prompt, then a hundred and fifty decoded one by one with given ids: every window passes over
    decoded tokens, pages fill and (in windowed groups) go back, the filters' and the bigram's state is carried
    through every step."""
    folder, cfg, w = models["S"]
    toks = random_tokens(153, cfg["vocab"], seed=8)
    steps = tail_trace({"long": toks}, 150)
    got = run_trace_engine(folder, dtype, steps, 192, PAGE_SIZES["S"])
    worst, where = worst_diff(got, plain_rows(cfg, w, {"long": toks}))
    assert worst <= tol("S", dtype), (worst, where)
