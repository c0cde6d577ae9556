"""Veredra through the engine against the plain implementation (`plain_veredra.py`): every mechanism alone,
whole prompts, portions, token-by-token decoding, unequal batches, reused slots and pages, window edges,
far keys, long decoding, other sizes, generation through the entry point, and the replay tool."""
from __future__ import annotations

import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_veredra as P
import veredra_tiny as V

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TOL = {"float32": 2e-4, "bfloat16": 3e-2}


def err(got, want, rms=False):
    """Difference of two sets of logit rows, mean taken off, relative to the spread of the expected row: the
    largest element of the worst row (the sharp measure, for float32).  With `rms` (bfloat16, whose rounding is
    judged by its size): the root mean square of a row, and of the rows the one that nine in ten stay under; the
    worst row (a position where a near-tie in a softmax multiplies every rounding, in float32 just as much) may be
    four times that."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    size = (d.pow(2).mean(-1).sqrt() if rms else d.abs().max(-1).values) / w.pow(2).mean(-1).sqrt().clamp_min(1e-6)
    if rms:
        return max(torch.quantile(size, 0.9).item(), size.max().item() / 4)
    return size.max().item()


class Built:
    """A configuration with weights: the model folder, the plain logits per request (cached)."""

    def __init__(self, cfg, seed, tmp, decay_rank=8):
        self.cfg, self.W = cfg, V.draw_weights(cfg, seed, decay_rank)
        self.dir = V.write_model(cfg, self.W, root=str(tmp))
        self._plain = {}

    def plain(self, toks):
        key = tuple(toks)
        if key not in self._plain:
            self._plain[key] = P.forward(self.cfg, self.W, list(toks))
        return self._plain[key]

    def engine(self, dtype, **kw):
        from cpi_b200.engine import Engine
        kw.setdefault("max_tokens", 4096)
        return Engine.from_model_dir(self.dir, dtype=dtype, **kw)


class Run:
    """Feeds requests to an engine step by step and keeps the logits by (request, position)."""

    def __init__(self, engine):
        self.e, self.slots, self.logits = engine, {}, {}

    def step(self, items):
        from cpi_b200.engine import StepEntry
        entries, layout = [], []
        for rid, toks, want in items:
            if rid not in self.slots:
                self.slots[rid] = self.e.acquire_slot()
            start = self.e.length(self.slots[rid])
            entries.append(StepEntry(self.slots[rid], list(toks), list(want)))
            layout.append((rid, start, list(want)))
        out = self.e.step(entries).float().cpu()
        self.e.check_device_errors()
        r = 0
        for rid, start, want in layout:
            for w in want:
                self.logits.setdefault(rid, {})[start + w] = out[r]
                r += 1

    def end(self, rid):
        self.e.release_slot(self.slots.pop(rid))

    def check(self, built, requests, tol):
        worst = 0.0
        for rid, got in self.logits.items():
            ref = built.plain(requests[rid])
            pos = sorted(got)
            e = err(torch.stack([got[p] for p in pos]), ref[pos], rms=tol > 1e-3)
            assert e < tol, f"request {rid}: error {e:.3g} (tolerance {tol}) over positions {pos[0]}..{pos[-1]}"
            worst = max(worst, e)
        return worst


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("veredra")
    return {"A": Built(V.MIXED_A, 11, tmp), "B": Built(V.MIXED_B, 12, tmp, decay_rank=5),
            "C": Built(V.MIXED_C, 13, tmp, decay_rank=16), "D": Built(V.GLA_ONLY, 14, tmp, decay_rank=3)}


# ---- kernels alone ---------------------------------------------------------------------------------------
def K():
    from cpi_b200.csrc import lib
    return lib


class FakeBatch:
    """The index arrays a kernel reads of a step: sequences of `n_new` tokens that start at `starts`."""

    def __init__(self, slots, starts, n_new, dev):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        self.n_seqs, self.max_new = len(slots), max(n_new)
        self.seq_slot, self.seq_start, self.seq_new = i32(slots), i32(starts), i32(n_new)
        tok0, seq, pos, base = [], [], [], 0
        for s, (st, n) in enumerate(zip(starts, n_new)):
            tok0.append(base); seq += [s] * n; pos += range(st, st + n); base += n
        self.seq_tok0, self.token_seq, self.token_pos = i32(tok0), i32(seq), i32(pos)


@pytest.mark.parametrize("S,Wd", [(1, 100), (2, 100), (3, 2048), (5, 100), (8, 5000)])
def test_stream_mixing_kernel(S, Wd):
    """Write-back of one sublayer and read of the next: x_t <- sum_s M[s, t] x_s + b[t] y, u = sum_s a[s] x_s,
    h = u * rsqrt(mean u^2 + eps) * (1 + w); then the read alone over chosen rows.  Narrow rows, rows that fill the
    largest block once, and rows wider than a block's registers hold."""
    dev, T = "cuda", 7
    g = torch.Generator().manual_seed(S)
    x = torch.randn(S, T, Wd, generator=g).to(dev)
    y, mix, write, read = (torch.randn(*s, generator=g).to(dev) for s in ((T, Wd), (S, S), (S,), (S,)))
    w = (torch.randn(Wd, generator=g) * 0.2).to(torch.bfloat16).to(dev)
    x_new = torch.einsum("st,snw->tnw", mix.double(), x.double()) + write.double()[:, None, None] * y.double()[None]
    u = torch.einsum("s,snw->nw", read.double(), x_new)
    h_ref = P.norm_one_plus(u, w.double(), 1e-5)
    h = torch.empty(T, Wd, device=dev)
    xk = x.clone()
    K().hc_step(xk, y=y, mix=mix, write=write, read=read, norm_weight=w, norm_offset=1.0, eps=1e-5, h_out=h)
    assert (xk.double() - x_new).abs().max() < 1e-5 and (h.double() - h_ref).abs().max() < 1e-4
    rows = torch.tensor([5, 0, 5, 2], dtype=torch.int32, device=dev)
    h2, s2 = torch.empty(4, Wd, device=dev, dtype=torch.bfloat16), torch.empty(4, Wd, device=dev)
    before = xk.clone()
    K().hc_step(xk, rows=rows, norm_weight=w, norm_offset=1.0, eps=1e-5, h_out=h2, sum_out=s2)
    total = x_new.sum(0)[rows.long()]
    assert (s2.double() - total).abs().max() < 1e-5
    assert (h2.double() - P.norm_one_plus(total, w.double(), 1e-5)).abs().max() < 3e-2
    assert torch.equal(xk, before)                                         # the read changes nothing


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_causal_convolution_with_carried_inputs(taps):
    """Two sequences whose tokens come as 5 + 1 + 3 and 2 + 1 + 1: the result is that of the whole sequences."""
    dev, C = "cuda", 37
    g = torch.Generator().manual_seed(taps)
    n_total = [9, 4]
    xs = [torch.randn(n, C, generator=g) for n in n_total]
    w, b = torch.randn(C, taps, generator=g).to(torch.bfloat16), torch.randn(C, generator=g).to(torch.bfloat16)
    ref = [P.silu(P.causal_conv(x.double(), w.double(), b.double())) for x in xs]
    carry = torch.full((4, max(taps - 1, 0), C), 7.0, device=dev)          # slots 3 and 1 are used; stale values
    carry[3].zero_(); carry[1].zero_()
    done = [0, 0]
    for cut in ([5, 2], [1, 1], [3, 1]):
        fb = FakeBatch([3, 1], done, cut, dev)
        x = torch.cat([xs[s][done[s]:done[s] + cut[s]] for s in range(2)]).to(dev)
        wide = torch.zeros(x.shape[0], C + 6, device=dev)                  # a column slice of a wider row
        wide[:, 3:3 + C] = x
        out = torch.empty(x.shape[0], C, device=dev)
        K().causal_conv(wide[:, 3:3 + C], w.to(dev), b.to(dev), carry, out, fb, silu=True)
        want = torch.cat([ref[s][done[s]:done[s] + cut[s]] for s in range(2)])
        assert (out.cpu().double() - want).abs().max() < 1e-5
        done = [d + c for d, c in zip(done, cut)]


@pytest.mark.parametrize("rows,cols,heads,per_group", [(24, 20, 6, 2), (64, 33, 2, 1), (130, 16, 3, 3), (8, 5, 4, 4),
                                                       (96, 12, 2, 2), (200, 9, 1, 1), (300, 8, 2, 1), (600, 4, 1, 1)])
def test_recurrence_kernel_both_flavours(rows, cols, heads, per_group):
    """S_t = diag(a_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t over a sequence cut as 20 + 1 + 1 + 6 + 18 beside a second
    one, with a decay per row (sigmoid(z + b)^(1/tau)) and with a decay per head (softplus step, skip term).  Long
    portions take the kernel's wide blocks and short ones its narrow blocks, on the same state."""
    dev, n = "cuda", 46
    g = torch.Generator().manual_seed(rows)
    groups = heads // per_group
    k, q = torch.randn(n, groups * rows, generator=g), torch.randn(n, groups * rows, generator=g)
    v = torch.randn(n, heads * cols, generator=g)
    z, zb = torch.randn(n, heads * rows, generator=g), torch.randn(heads * rows, generator=g) + 2
    dt, dtb = torch.randn(n, heads, generator=g), torch.randn(heads, generator=g)
    a_log, skip = torch.randn(heads, generator=g) - 1, torch.randn(heads, generator=g)

    def plain(row_decay):
        out = torch.zeros(n, heads, cols, dtype=torch.float64)
        for h in range(heads):
            gi = h // per_group
            S = torch.zeros(rows, cols, dtype=torch.float64)
            for t in range(n):
                kt, qt = k[t, gi * rows:(gi + 1) * rows].double(), q[t, gi * rows:(gi + 1) * rows].double()
                vt = v[t, h * cols:(h + 1) * cols].double()
                if row_decay:
                    a = torch.exp(torch.nn.functional.logsigmoid(z[t, h * rows:(h + 1) * rows].double()
                                                                 + zb[h * rows:(h + 1) * rows].double()) / 4.0)
                    S = a[:, None] * S + torch.outer(kt, vt)
                    out[t, h] = S.T @ (qt * 0.5)
                else:
                    step = P.softplus(dt[t, h].double() + dtb[h].double())
                    S = torch.exp(-torch.exp(a_log[h].double()) * step) * S + step * torch.outer(kt, vt)
                    out[t, h] = S.T @ qt + skip[h].double() * vt
        return out.reshape(n, heads * cols)

    for row_decay in (True, False):
        ref = plain(row_decay)
        state = torch.full((3, heads, rows, cols), 3.0, device=dev)
        state[2].zero_(); state[0].zero_()
        done = 0
        for cut in (20, 1, 1, 6, 18):
            fb = FakeBatch([2, 0], [done, done], [cut, cut], dev)          # the same sequence twice, in two slots
            sl = slice(done, done + cut)
            two = lambda t: torch.cat([t[sl], t[sl]]).to(dev).contiguous()
            out = torch.empty(2 * cut, heads * cols, device=dev)
            kw = dict(n_heads=heads, heads_per_group=per_group, n_rows=rows, n_cols=cols)
            if row_decay:
                before = state.clone()
                K().linear_scan(two(k), two(q), two(v), state, out, fb, z=two(z), z_bias=zb.to(dev), tau=4.0, q_scale=0.5, **kw)
                # decays prepared by their own kernel: the same bits in the outputs and in the state
                a, out2 = two(z), torch.empty_like(out)
                K().row_decay(a, zb.to(dev), 4.0)
                want_a = torch.exp(torch.nn.functional.logsigmoid(two(z).double() + zb.to(dev).double()) / 4.0)
                assert (a.double() - want_a).abs().max() < 1e-6
                K().linear_scan(two(k), two(q), two(v), before, out2, fb, z=a, tau=4.0, q_scale=0.5, decay_ready=True, **kw)
                assert torch.equal(out, out2) and torch.equal(state, before)
            else:
                K().linear_scan(two(k), two(q), two(v), state, out, fb, dt=two(dt), dt_bias=dtb.to(dev),
                                a_log=a_log.to(dev), skip=skip.to(dev), **kw)
            got = out.cpu().double()
            scale = ref.abs().max()
            assert (got[:cut] - ref[sl]).abs().max() < 2e-5 * scale and torch.equal(got[:cut], got[cut:])
            done += cut
        assert torch.equal(state[1], torch.full_like(state[1], 3.0))       # a slot that no sequence holds is not touched


def test_gated_norm_gelu_gate_and_logit_cap_kernels():
    dev = "cuda"
    g = torch.Generator().manual_seed(5)
    y, gate = torch.randn(6, 60, generator=g).to(dev), torch.randn(6, 60, generator=g).to(dev)
    w, w_shared = torch.randn(60, generator=g).to(dev), torch.randn(15, generator=g).to(dev)
    out = torch.empty(6, 60, device=dev)
    K().gated_norm(y, gate, w, out, parts=3, gate_first=True, eps=1e-5)
    ref = P.rms_unit((y.double() * P.silu(gate.double())).view(6, 3, 20), 1e-5).reshape(6, 60) * w.double()
    assert (out.double() - ref).abs().max() < 1e-5
    K().gated_norm(y, gate, w_shared, out, parts=4, gate_first=False, eps=1e-5)
    ref = (P.rms_unit(y.double().view(6, 4, 15), 1e-5) * w_shared.double()).reshape(6, 60) * P.silu(gate.double())
    assert (out.double() - ref).abs().max() < 1e-5
    gu = torch.randn(5, 2 * 33, generator=g).to(dev) * 3
    a = torch.empty(5, 33, device=dev)
    K().gated_act(gu, a, "gelu_tanh")
    assert (a.double() - P.gelu_tanh(gu[:, :33].double()) * gu[:, 33:].double()).abs().max() < 1e-5
    lg = torch.randn(4, 50, generator=g).to(dev) * 40
    ref = 9.0 * torch.tanh(lg.double() * 0.5 / 9.0)
    K().logit_post(lg, 0.5, 9.0)
    assert (lg.double() - ref).abs().max() < 1e-5


@pytest.mark.parametrize("T,I,H,dtype", [(5, 72, 40, torch.float32), (40, 200, 136, torch.bfloat16),
                                         (600, 256, 128, torch.bfloat16)])
def test_gelu_gate_in_the_product_epilogue(T, I, H, dtype):
    """out = gelu_tanh(h Wg^T) * (h Wu^T) from one product over [Wg; Wu], on the float32 pipe, on the tensor-core
    kernel and on the paired kernel (many tokens, features a multiple of 256)."""
    from cpi_b200.parts.linear import MODE_GEGLU, project
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, H, generator=g).to(dtype).cuda()
    w = (torch.randn(2 * I, H, generator=g) * H ** -0.5 * 2).to(torch.bfloat16).cuda()
    out = torch.empty(T, I, dtype=dtype, device="cuda")
    project(h, w, out, MODE_GEGLU)
    gu = h.double() @ w.double().T
    ref = P.gelu_tanh(gu[:, :I]) * gu[:, I:]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out.double() - ref).abs().max() < tol * ref.abs().max()


def _sink_reference(q, k, v, pos, lo, scale, sink):
    """q [NH, D] at position `pos` over keys lo..pos of k, v [n, NKV, D]; exp(sink[h]) joins the denominator."""
    q, k, v, sink = q.cpu(), k.cpu(), v.cpu(), sink.cpu()
    NH, G = q.shape[0], q.shape[0] // k.shape[1]
    out = torch.empty(NH, v.shape[-1], dtype=torch.float64)
    for h in range(NH):
        sc = (k[lo:pos + 1, h // G].double() @ q[h].double()) * scale
        top = max(sc.max().item(), sink[h].item())
        e = torch.exp(sc - top)
        out[h] = (e / (e.sum() + math.exp(sink[h].item() - top))) @ v[lo:pos + 1, h // G].double()
    return out


@pytest.mark.parametrize("NH,NKV,D,window", [(8, 2, 128, ("sliding", 130)), (6, 6, 64, ("sliding", 64)),
                                             (4, 1, 64, ("full", 0))])
def test_sink_in_all_three_attention_kernels(NH, NKV, D, window):
    """A sink per head, from far below the scores to far above them, in the general kernel, in the tensor-core
    decode kernel (one split and several) and in the tensor-core prefill kernel."""
    import test_gpu_kernels as TK
    page, (wk, wsz), scale = 64, window, 1.0 / math.sqrt(D)
    sink = (torch.linspace(-6.0, 9.0, NH) + 0.3).cuda()
    low = lambda pos: 0 if wk == "full" else max(0, pos - wsz + 1)
    lengths = [1, 64, 65, 500, 129]
    k, v, table = TK.paged_cache(len(lengths), lengths, NKV, D, page, torch.bfloat16, seed=3)
    T = len(lengths)
    q = TK.rnd(T, NH * D, dtype=torch.bfloat16, seed=4)
    token_seq = torch.arange(T, dtype=torch.int32, device="cuda")
    token_pos = torch.tensor([l - 1 for l in lengths], dtype=torch.int32, device="cuda")
    seq_slot = torch.arange(1, T + 1, dtype=torch.int32, device="cuda")
    kw = dict(n_heads=NH, n_kv_heads=NKV, head_dim=D, window_kind=K().WINDOW_KINDS[wk], window_size=wsz, scale=scale)
    refs = []
    for i, l in enumerate(lengths):
        kk, vv = TK.gather_kv(k, table, i + 1, l, page), TK.gather_kv(v, table, i + 1, l, page)
        refs.append(_sink_reference(q[i].float().view(NH, D), kk, vv, l - 1, low(l - 1), scale, sink).reshape(-1))
    outs = {}
    outs["general"] = torch.empty_like(q)
    K().attention_general(q, outs["general"], k, v, table, page, token_seq, token_pos, seq_slot, sink=sink, **kw)
    for splits in (1, 5):
        outs[f"decode{splits}"] = torch.empty_like(q)
        K().attention_decode(q, outs[f"decode{splits}"], k, v, table, page, token_seq, token_pos, seq_slot,
                             n_splits=splits, sink=sink, **kw)
    for name, out in outs.items():
        for i in range(T):
            e = (out[i].double().cpu() - refs[i]).abs().max().item()
            assert e <= 1.5e-2 * max(1.0, refs[i].abs().max().item()), (name, i, e)
    c = TK._prefill_case(NH, NKV, D, window, [(0, 1), (0, 300), (70, 200), (100, 140)], tile=256)
    out = torch.full_like(c["q"], float("nan"))
    K().attention_prefill(c["q"], out, c["k"], c["v"], c["table"], page, c["token_seq"], c["token_pos"], c["seq_slot"],
                          c["tile_tok0"], c["tile_rows"], sink=sink, **kw)
    torch.cuda.synchronize()
    kk = [TK.gather_kv(torch.nan_to_num(c["k"]), c["table"], i + 1, l, page) for i, l in enumerate(c["lengths"])]
    vv = [TK.gather_kv(torch.nan_to_num(c["v"]), c["table"], i + 1, l, page) for i, l in enumerate(c["lengths"])]
    for t, (sq, pos) in enumerate(zip(c["seq"], c["pos"])):
        ref = _sink_reference(c["q"][t].float().view(NH, D), kk[sq], vv[sq], pos, low(pos), scale, sink).reshape(-1)
        e = (out[t].double().cpu() - ref).abs().max().item()
        assert e <= 1.5e-2 * max(1.0, ref.abs().max().item()), ("prefill", t, sq, pos, e)


# ---- each mixer alone, as a one-layer model --------------------------------------------------------------
ALONE = {
    "attention_window_sink": V.model([V.attention(4, 2, 24, 40, window=9, rot_dims=12)], 56, 90),
    "attention_full_no_rotation": V.model([V.attention(3, 3, 16, 16)], 48, 90),
    "attention_one_head_whole_rotation": V.model([V.attention(1, 1, 64, 8, window=33, rot_dims=64)], 40, 90),
    "mamba2": V.model([V.mamba2(4, 12, 20, 2, 3, 2)], 56, 90),
    "mamba2_one_tap": V.model([V.mamba2(2, 40, 8, 2, 1, 1)], 56, 90),
    "gla": V.model([V.gla(3, 20, 28, 4.0)], 56, 90),
    "mlp_and_streams": V.model([V.with_mlp(V.gla(1, 8, 8, 1.0), 72)], 56, 90, streams=2, softcap=5.0, logit_scale=3.0),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_prefill_and_decoding(name, tmp_path):
    """A model of one layer: whole prompt in float32 and bfloat16, and the same prompt cut as 17 tokens, a portion
    of 2, a portion of 9, then token by token."""
    b = Built(ALONE[name], 3, tmp_path)
    toks = V.tokens(60, 90, 1)
    for dtype in ("float32", "bfloat16"):
        r = Run(b.engine(dtype))
        r.step([("w", toks, range(60))])
        r.end("w")
        r.step([("c", toks[:17], range(17))])
        r.step([("c", toks[17:19], range(2))])
        r.step([("c", toks[19:28], range(9))])
        for i in range(28, 60):
            r.step([("c", toks[i:i + 1], [0])])
        r.check(b, {"w": toks, "c": toks}, TOL[dtype])
        if dtype == "float32":       # how the prompt was cut changes nothing beyond rounding
            assert err(torch.stack([r.logits["c"][p] for p in range(60)]),
                       torch.stack([r.logits["w"][p] for p in range(60)])) < 5e-5


# ---- schedules on the mixed models ----------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16"),
                                        ("C", "float32"), ("C", "bfloat16"), ("D", "float32")])
def test_whole_prompts_and_token_by_token(models, name, dtype):
    b = models[name]
    vocab = b.cfg["vocab"]
    reqs = {"long": V.tokens(150, vocab, 1), "one": V.tokens(1, vocab, 2), "two": V.tokens(2, vocab, 3)}
    r = Run(b.engine(dtype))
    for rid, toks in reqs.items():
        r.step([(rid, toks, range(len(toks)))])
        r.end(rid)
    r.check(b, reqs, TOL[dtype])
    r = Run(b.engine(dtype))
    toks = reqs["long"]
    r.step([("long", toks[:90], [0, 1, 2, 89])])          # the first tokens of a sequence, then decoding
    for i in range(90, 150):
        r.step([("long", toks[i:i + 1], [0])])
    r.check(b, reqs, TOL[dtype])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_several_sizes(models, name):
    """A prompt in portions of 2, 3, 64, 1, 61, 70 and 30 tokens (cuts inside pages and windows), logits on both
    sides of every cut; with a small step limit the engine cuts the portions itself once more."""
    b = models[name]
    toks = V.tokens(231, b.cfg["vocab"], 4)
    for limit in (8192, 37):
        r = Run(b.engine("float32", max_step_tokens=limit))
        at = 0
        for n in (2, 3, 64, 1, 61, 70, 30):
            r.step([("p", toks[at:at + n], sorted({0, n - 1, n // 2}))])
            at += n
        r.check(b, {"p": toks}, TOL["float32"])


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("C", "bfloat16")])
def test_unequal_batches_in_reused_slots(models, name, dtype):
    """Groups of unequal requests start together and go on by one token each, the shorter ending earlier; group
    follows group in a cache with room for one group, so slots, pages and states are used again."""
    b = models[name]
    vocab = b.cfg["vocab"]
    lens = [131, 7, 64, 1, 90, 65, 3, 128]
    reqs = {f"r{i}": V.tokens(n + 20, vocab, 10 + i) for i, n in enumerate(lens)}
    eng = b.engine(dtype, max_tokens=4 * 192, max_seqs=4)
    r = Run(eng)
    for g0 in range(0, len(lens), 4):
        group = [f"r{i}" for i in range(g0, g0 + 4)]
        head = {rid: len(reqs[rid]) - 20 - (5 if rid.endswith(("1", "6")) else 0) for rid in group}
        head = {rid: max(1, h) for rid, h in head.items()}
        r.step([(rid, reqs[rid][:head[rid]], [head[rid] - 1]) for rid in group])
        k = 0
        live = list(group)
        while live:
            r.step([(rid, [reqs[rid][head[rid] + k]], [0]) for rid in live])
            k += 1
            for rid in [x for x in live if head[x] + k >= len(reqs[x])]:
                r.end(rid)
                live.remove(rid)
        eng.cache.check_consistency()
    r.check(b, reqs, TOL[dtype])
    # each alone in a fresh engine gives the batch's logits (float32: to rounding)
    if dtype == "float32":
        alone = Run(b.engine(dtype))
        rid = "r4"
        h = len(reqs[rid]) - 20
        alone.step([(rid, reqs[rid][:h], [h - 1])])
        for i in range(h, len(reqs[rid])):
            alone.step([(rid, [reqs[rid][i]], [0])])
        pos = sorted(alone.logits[rid])
        assert err(torch.stack([r.logits[rid][p] for p in pos]), torch.stack([alone.logits[rid][p] for p in pos])) < 5e-5


def test_a_key_just_inside_and_just_outside_the_window(tmp_path):
    """One attention layer and nothing else, so that the last token's logits depend on exactly the keys of its
    window.  A token is replaced at distance window - 1 (the last one seen) and at distance window (the first one
    not seen): the first changes the answer, the second leaves it as it was, and the engine agrees with the plain
    implementation both times, in a prompt and in decoding, with the edge at a page border and inside a page."""
    for window, n in ((17, 64 + 17 + 3), (64, 200), (5, 9)):
        cfg = V.model([V.attention(2, 1, 32, 32, window=window, rot_dims=8)], 32, 50)
        b = Built(cfg, window, tmp_path)
        base = V.tokens(n, 49, window)                      # token 49 is the marked one
        seen = {}
        for dist in (window - 1, window):
            toks = list(base)
            toks[n - 1 - dist] = 49
            ref = b.plain(toks)
            for mode in ("prompt", "decode"):
                r = Run(b.engine("float32"))
                if mode == "prompt":
                    r.step([("x", toks, [n - 1])])
                else:
                    cut = max(1, n - window - 2)
                    r.step([("x", toks[:cut], [])])
                    for i in range(cut, n):
                        r.step([("x", toks[i:i + 1], [0] if i == n - 1 else [])])
                assert err(r.logits["x"][n - 1][None], ref[n - 1][None]) < TOL["float32"], (window, dist, mode)
            seen[dist] = ref[n - 1]
        plain_base = b.plain(base)[n - 1]
        # the marked token matters inside the window and not at all outside it
        assert err(seen[window][None], plain_base[None]) < 1e-9 < 1e-3 < err(seen[window - 1][None], plain_base[None])


def test_a_far_token_among_hundreds(models):
    """Models whose recurrent layers keep state for hundreds of tokens and whose last attention layer sees all keys:
    changing one early token changes late logits, and the engine follows the plain implementation there, in one
    step, in portions and decoded."""
    b = models["A"]
    vocab = b.cfg["vocab"]
    toks = V.tokens(520, vocab, 8)
    other = list(toks)
    other[3] = (toks[3] + 1) % vocab
    late = [400, 470, 519]
    assert err(b.plain(other)[late], b.plain(toks)[late]) > 1e-3           # the far token is felt
    r = Run(b.engine("float32"))
    r.step([("whole", other, late)])
    r.step([("cut", other[:129], [])])
    r.step([("cut", other[129:450], [400 - 129])])
    for i in range(450, 520):
        r.step([("cut", other[i:i + 1], [0] if i in late else [])])
    r.check(b, {"whole": other, "cut": other}, TOL["float32"])


def test_long_decoding_past_windows_and_pages(models):
    """300 tokens one by one after a prompt of 3: windows of 5 and 70 slide over decoded tokens and page borders,
    the window groups give pages back."""
    b = models["B"]
    toks = V.tokens(303, b.cfg["vocab"], 9)
    eng = b.engine("float32", max_tokens=512)
    r = Run(eng)
    r.step([("d", toks[:3], [2])])
    for i in range(3, 303):
        r.step([("d", toks[i:i + 1], [0])])
    r.check(b, {"d": toks}, TOL["float32"])
    windowed = [g for g in eng.cache.groups if g.req.window_kind == "sliding"]
    assert windowed and all(g.pages_held() <= 3 for g in windowed)


def test_other_constants_change_the_result_as_the_plain_implementation_says(tmp_path):
    """Values that one model may happen to make equal or 1: streams, loop, scale, tau, eps, window, rotation base,
    norm groups, softcap.  Each is changed alone and the engine follows."""
    base = V.model([V.with_mlp(V.attention(2, 1, 16, 24, window=6, rot_dims=16), 40),
                    V.with_mlp(V.mamba2(4, 8, 12, 2, 3, 2), 40), V.with_mlp(V.gla(2, 12, 8, 4.0), None)],
                   48, 70, streams=2, loop=(0, 2, 2), logit_scale=0.9, softcap=20.0)
    import copy
    variants = {"base": base}
    for key, change in {
        "streams": lambda c: c.update(streams=3), "no_loop": lambda c: c.pop("loop"),
        "loop_late": lambda c: c.update(loop={"start": 1, "stop": 3, "times": 3}),
        "scale": lambda c: c["layers"][0]["mixer"].update(scale=1.1), "tau": lambda c: c["layers"][2]["mixer"].update(tau=1.5),
        "eps": lambda c: c.update(norm={"eps": 0.3}), "window": lambda c: c["layers"][0]["mixer"].update(mask={"size": 7}),
        "base": lambda c: c["layers"][0]["mixer"]["rot"].update(base=77.0),
        "rot_dims": lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6),
        "norm_groups": lambda c: c["layers"][1]["mixer"].update(norm_groups=4),
        "groups": lambda c: c["layers"][1]["mixer"].update(groups=4),
        "kv_heads": lambda c: c["layers"][0]["mixer"].update(kv_heads=2),
        "no_cap": lambda c: c.pop("logit_softcap"), "logit_scale": lambda c: c.update(logit_scale=2.0),
    }.items():
        c = copy.deepcopy(base)
        change(c)
        variants[key] = c
    toks = V.tokens(40, 70, 2)
    for key, cfg in variants.items():
        b = Built(cfg, 21, tmp_path)
        r = Run(b.engine("float32"))
        r.step([("x", toks[:25], range(25))])
        for i in range(25, 40):
            r.step([("x", toks[i:i + 1], [0])])
        r.check(b, {"x": toks}, TOL["float32"])


def test_greedy_generation_through_the_entry_point(models):
    """`Model.generate` (scheduler, sampler, decode graphs) picks the plain implementation's tokens: unequal
    prompts, more requests than slots."""
    from cpi_b200.api import Model
    b = models["A"]
    vocab = b.cfg["vocab"]
    prompts = [V.tokens(n, vocab, 30 + n) for n in (5, 33, 1, 70, 12)]
    m = Model.load(b.dir, dtype="float32", max_batch=2, max_context=128)
    results = m.generate(prompts, max_new=12, temperature=0.0)
    for p, res in zip(prompts, results):
        seq = list(p)
        for tok in res.tokens:
            ref = b.plain(seq)[-1]
            best = int(ref.argmax())
            if tok != best:            # a near-tie may fall either way; anything else is a fault
                assert (ref[best] - ref[tok]).item() < 1e-3 * ref.abs().max().item(), (len(p), len(seq))
            seq.append(tok)
        assert len(res.tokens) == 12


def test_command_line_generates_with_a_veredra_folder(models):
    """bin/llama_infer knows the family by its config.json: greedy tokens are the plain implementation's, and the
    phase report names the recurrent mixers' phases."""
    b = models["C"]
    prompt = V.tokens(9, b.cfg["vocab"], 50)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llama_infer"), b.dir, "--tokens",
                        ",".join(map(str, prompt)), "--max-new", "6", "--temp", "0", "--dtype", "float32",
                        "--benchmark-phases", "--max-context", "64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = next(l for l in r.stdout.splitlines() if l.startswith("Output tokens:"))
    got = [int(x) for x in line.split(":")[1].split()]
    assert got[:9] == prompt and len(got) == 15
    seq = list(prompt)
    for tok in got[9:]:
        ref = b.plain(seq)[-1]
        best = int(ref.argmax())
        assert tok == best or (ref[best] - ref[tok]).item() < 1e-3 * ref.abs().max().item()
        seq.append(tok)
    assert "Veredra" in r.stdout and "scan" in r.stdout


def test_replay_tool_runs_a_veredra_folder(models, tmp_path):
    """bin/trace_run in a process of its own: a request whole, and two requests batched then decoded."""
    b = models["B"]
    vocab = b.cfg["vocab"]
    ta, tb = V.tokens(80, vocab, 40), V.tokens(21, vocab, 41)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ta, "want": [0, 79]}], "end": ["a"]},
             {"step": 1, "entries": [{"id": "b", "tokens": tb[:20], "want": []},
                                     {"id": "a2", "tokens": ta[:70], "want": [69]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": tb[20:], "want": [0]},
                                     {"id": "a2", "tokens": ta[70:71], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a2", "tokens": ta[71:72], "want": [0]}], "end": ["a2"]}]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / f"out_{dtype}"
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", b.dir, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps),
                           capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
        import numpy as np
        rd = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab).copy())
        ra, rb = b.plain(ta), b.plain(tb)
        rms = dtype == "bfloat16"
        assert err(rd(0), ra[[0, 79]], rms) < TOL[dtype]
        assert err(rd(1), ra[[69]], rms) < TOL[dtype]
        assert err(rd(2), torch.stack([rb[20], ra[70]]), rms) < TOL[dtype]
        assert err(rd(3), ra[[71]], rms) < TOL[dtype]
