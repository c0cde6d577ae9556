"""Savenex through the engine against the plain implementation (`plain_savenex.py`): every mechanism alone, whole
prompts, portions, token-by-token decoding, unequal batches, reused slots and pages, the edges of windows and of the
kept first tokens, far keys, long decoding, other sizes, generation through the entry point, and the replay tool."""
from __future__ import annotations

import copy
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import plain_savenex as P
import savenex_tiny as V

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
F64 = torch.float64


def err(got, want, rms=False):
    """Difference of logit rows, mean taken off, relative to the spread of the expected row: the largest element of the
    worst row (float32), or with `rms` (bfloat16) a row's root mean square: what nine rows in ten stay under, and a
    quarter of the worst row.  In bfloat16 a router's near-tie may choose another expert than the plain implementation
    does, which is no fault and changes that position's logits wholesale: of five rows or more, the worst one in fifty
    (at least one) is left out of the second measure."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    size = (d.pow(2).mean(-1).sqrt() if rms else d.abs().max(-1).values) / w.pow(2).mean(-1).sqrt().clamp_min(1e-6)
    if rms:
        n = size.numel()
        drop = max(1, math.ceil(0.02 * n)) if n >= 5 else 0
        kept = size.sort().values[:n - drop]
        return max(torch.quantile(size, 0.9).item(), kept.max().item() / 4)
    return size.max().item()


class Built:
    def __init__(self, cfg, seed, tmp, ranks=(6, 5)):
        self.cfg, self.W = cfg, V.draw_weights(cfg, seed, ranks)
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
        for rid, got in self.logits.items():
            ref = built.plain(requests[rid])
            pos = sorted(got)
            e = err(torch.stack([got[p] for p in pos]), ref[pos], rms=tol > 1e-3)
            assert e < tol, f"request {rid}: error {e:.3g} (tolerance {tol}) over positions {pos[0]}..{pos[-1]}"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("savenex")
    return {"A": Built(V.MIXED_A, 11, tmp), "B": Built(V.MIXED_B, 12, tmp, ranks=(16, 8)),
            "C": Built(V.MIXED_C, 13, tmp, ranks=(3, 1))}


def K():
    from cpi_b200.csrc import lib
    return lib


class FakeBatch:
    """The index arrays a kernel reads of a step: sequences of `n_new` tokens that start at `starts`."""

    def __init__(self, slots, starts, n_new, dev="cuda"):
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        self.n_seqs, self.max_new = len(slots), max(n_new)
        self.seq_slot, self.seq_start, self.seq_new = i32(slots), i32(starts), i32(n_new)
        tok0, seq, pos, base = [], [], [], 0
        for s, (st, n) in enumerate(zip(starts, n_new)):
            tok0.append(base); seq += [s] * n; pos += range(st, st + n); base += n
        self.seq_tok0, self.token_seq, self.token_pos = i32(tok0), i32(seq), i32(pos)


# ---- kernels alone ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols,heads,per_group", [(12, 20, 6, 2), (32, 64, 4, 1), (4, 20, 5, 1), (48, 24, 2, 2),
                                                       (128, 128, 2, 1), (64, 96, 3, 3), (10, 13, 2, 1), (200, 40, 2, 2)])
def test_delta_rule_recurrence_whole_in_pieces_and_token_by_token(rows, cols, heads, per_group):
    """The delta rule with a decay per key channel, against the token loop of the plain implementation: a prompt in
    one launch (prepared decays and decays made in the kernel), in pieces of several sizes down to one token, in a
    slot among others; the state after each is the plain one."""
    g = torch.Generator().manual_seed(rows * 7 + cols)
    T, groups = 45, heads // per_group
    rn = lambda *s, std=1.0, mean=0.0: (torch.randn(*s, generator=g) * std + mean)
    q, k = P.unit(rn(T, groups, rows).double()), P.unit(rn(T, groups, rows).double())
    v, beta_raw, z = rn(T, heads, cols), rn(T, heads, std=1.5), rn(T, heads * rows)
    a_log, bias = rn(heads, std=1.0, mean=-1.5), rn(heads * rows)
    decay = torch.exp(-torch.exp(a_log.double())[None, :, None] *
                      torch.nn.functional.softplus((z + bias).double()).view(T, heads, rows))
    qs = q.repeat_interleave(per_group, 1) * rows ** -0.5
    want = P.gated_delta(qs, k.repeat_interleave(per_group, 1), v.double(), torch.sigmoid(beta_raw.double()), decay)
    dev = "cuda"
    c = lambda t: t.float().to(dev).contiguous()
    kq = c(torch.cat([k.reshape(T, -1), q.reshape(T, -1)], 1))           # column slices, as the mixer passes them
    nk = groups * rows
    for cuts in ([T], [17, 1, 2, 25], [1] * T):
        for ready in (False, True):
            state = torch.zeros(3, heads, rows, cols, device=dev)
            out = torch.empty(T, heads * cols, device=dev)
            at = 0
            for n in cuts:
                b = FakeBatch([1], [at], [n])
                zz = c(z[at:at + n])
                if ready:
                    K().row_decay(zz, c(bias), 1.0, kind=1, a_log=c(a_log), rows_per_head=rows)
                K().linear_scan(kq[at:at + n, :nk], kq[at:at + n, nk:], c(v[at:at + n].reshape(n, -1)), state,
                                out[at:at + n], b, n_heads=heads, heads_per_group=per_group, n_rows=rows, n_cols=cols,
                                z=zz, z_bias=c(bias), a_log=c(a_log), decay_kind=1, decay_ready=ready,
                                q_scale=rows ** -0.5, beta=c(beta_raw[at:at + n]))
                at += n
            d = (out.cpu().double().view(T, heads, cols) - want).abs().max().item()
            assert d < 2e-5 * max(1.0, want.abs().max().item()), (cuts[:3], ready, d)
            assert state[0].abs().max().item() == 0 and state[2].abs().max().item() == 0


def test_unit_vectors_sigmoid_gated_norm_branch_sum_concat_and_clamped_gate_kernels():
    g = torch.Generator().manual_seed(3)
    dev, T = "cuda", 9
    x = torch.randn(T, 70, generator=g)
    buf = x.to(dev).clone()
    K().head_unit(buf[:, 10:70], heads=5, dim=12, eps=1e-6)              # a column slice: the first ten stay
    want = P.unit(x[:, 10:].double().view(T, 5, 12)).view(T, 60)
    assert (buf[:, 10:].cpu().double() - want).abs().max() < 1e-6 and torch.equal(buf[:, :10].cpu(), x[:, :10])
    y, gate, w = torch.randn(T, 60, generator=g), torch.randn(T, 60, generator=g), torch.randn(12, generator=g)
    out = torch.empty(T, 60, device=dev)
    K().gated_norm(y.to(dev), gate.to(dev), w.to(dev), out, parts=5, gate_first=False, eps=1e-5, gate_act="sigmoid")
    want = (P.rms_norm(y.double().view(T, 5, 12), w.double(), 1e-5) * torch.sigmoid(gate.double()).view(T, 5, 12)).view(T, 60)
    assert (out.cpu().double() - want).abs().max() < 1e-5
    a, b = torch.randn(T, 52, generator=g) * 3, torch.randn(T, 52, generator=g) * 0.1
    wa, wb = torch.randn(52, generator=g), torch.randn(52, generator=g)
    res = torch.randn(T, 52, generator=g)
    want = 0.5 * (P.rms_norm(a.double(), wa.double(), 1e-5) + P.rms_norm(b.double(), wb.double(), 1e-5))
    for add in (False, True):
        o = res.to(dev).clone()
        K().branch_norm_sum([a.to(dev), b.to(dev)], [wa.to(dev), wb.to(dev)], o, eps=1e-5, scale=0.5, add=add)
        assert (o.cpu().double() - (want + (res.double() if add else 0))).abs().max() < 1e-5
    for dt in (torch.float32, torch.bfloat16):
        cat = torch.empty(T, 104, dtype=dt, device=dev)
        K().concat_rows(a.to(dev), b.to(dev), cat)
        assert torch.equal(cat.cpu(), torch.cat([a, b], 1).to(dt))
    gu = torch.randn(T, 2 * 30, generator=g) * 3
    act = torch.empty(T, 30, device=dev)
    K().gated_act(gu.to(dev), act, "swish_clamped", 1.25)
    gg, uu = gu[:, :30].double().clamp(max=1.25), gu[:, 30:].double().clamp(-1.25, 1.25)
    assert (act.cpu().double() - gg * torch.sigmoid(1.702 * gg) * (uu + 1)).abs().max() < 1e-5


@pytest.mark.parametrize("T,I,H,dtype", [(5, 72, 40, torch.float32), (40, 200, 136, torch.bfloat16),
                                         (600, 256, 128, torch.bfloat16), (7, 96, 64, torch.bfloat16)])
def test_clamped_gate_in_the_product_epilogue(T, I, H, dtype):
    """out = g sigmoid(1.702 g) (u + 1), g = min(h Wg^T, limit), u = clamp(h Wu^T, -limit, limit), from one product
    over [Wg; Wu]: on the float32 pipe, on the tensor-core kernel and on the paired kernel (many tokens, features a
    multiple of 256); pre-activations a few limits wide, so that every clamp bites; also for experts in groups."""
    from cpi_b200.parts.linear import MODE_CLAMPED_GLU, project
    g = torch.Generator().manual_seed(T)
    limit = 1.25
    h = torch.randn(T, H, generator=g).to(dtype).cuda()
    w = (torch.randn(2 * I, H, generator=g) * H ** -0.5 * 3).to(torch.bfloat16).cuda()
    out = torch.empty(T, I, dtype=dtype, device="cuda")
    project(h, w, out, MODE_CLAMPED_GLU, gate_limit=limit)
    gu = h.double().cpu() @ w.double().cpu().T
    gg, uu = gu[:, :I].clamp(max=limit), gu[:, I:].clamp(-limit, limit)
    ref = gg * torch.sigmoid(1.702 * gg) * (uu + 1)
    assert (gu[:, :I] > limit).any() and (gu[:, I:] < -limit).any()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out.double().cpu() - ref).abs().max() < tol * ref.abs().max()


@pytest.mark.parametrize("T", [5, 300])
def test_router_with_a_bias_and_softmax_over_the_chosen(T):
    g = torch.Generator().manual_seed(T)
    dev, H, E, k = "cuda", 40, 7, 3
    h, w, b = torch.randn(T, H, generator=g), torch.randn(E, H, generator=g) * 0.3, torch.randn(E, generator=g) * 2
    i32, f32 = torch.int32, torch.float32
    idx, gate = torch.empty(T, k, dtype=i32, device=dev), torch.empty(T, k, device=dev)
    bufs = [torch.empty(n, dtype=d, device=dev) for n, d in ((T * E, f32), (E + 1, i32), (T * k, i32), (T * k, f32), (T * k, i32))]
    K().moe_route(h.to(dev), w.to(dev), idx, gate, bufs[0].view(T, E), bufs[1], bufs[2], bufs[3], bufs[4], top_k=k,
                  sigmoid_gate="softmax_chosen", bias=b.to(dev))
    z = h.double() @ w.double().T + b.double()
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:k]
        assert idx[t].tolist() == order
        assert (gate[t].cpu().double() - torch.softmax(z[t, order], 0)).abs().max() < 1e-5
    assert abs(gate.sum().item() - T) < 1e-3
    gates = torch.empty(T, E, device=dev)
    K().row_gates(h.to(dev), w.to(dev), gates, bias=b.to(dev))           # a gate per token and row, one launch
    assert (gates.cpu().double() - torch.sigmoid(z)).abs().max() < 1e-5


def test_kept_first_positions_in_the_attention_kernel():
    """One key is made to carry the row (its key is the query, the others are orthogonal to it): the output is that
    key's value exactly when the mask lets it through -- the last kept position and the first one not kept, the
    oldest key of the window and the one before it, in a prompt and for a single token, across a page border."""
    dev, D, Dv, page = "cuda", 16, 8, 64
    window, keep = 10, 67                                   # the kept range ends three positions into the second page
    n_pos = 200
    kc = torch.zeros(8, 1, page, D, device=dev)
    vc = torch.zeros(8, 1, page, Dv, device=dev)
    table = torch.tensor([[5, 2, 7, 1, 0, 0, 0, 0]], dtype=torch.int32, device=dev)
    pos_of = lambda p: (int(table[0, p // page]), p % page)
    for p in range(n_pos):
        pg, off = pos_of(p)
        kc[pg, 0, off, 1 + p % (D - 1)] = 1.0               # orthogonal to the query direction (element 0)
        vc[pg, 0, off] = torch.full((Dv,), float(p + 1))
    for target, qpos, seen in ((66, 190, True), (67, 190, False), (67, 76, True), (66, 199, True), (181, 190, True),
                               (180, 190, False), (0, 199, True), (189, 199, False), (190, 199, True)):
        pg, off = pos_of(target)
        old = kc[pg, 0, off].clone()
        kc[pg, 0, off] = 0
        kc[pg, 0, off, 0] = 1.0
        for n_q in (1, 3):                                  # a single token; the last of a portion of three
            first = qpos - n_q + 1
            q = torch.zeros(n_q, D, device=dev)
            q[:, 0] = 40.0
            b = FakeBatch([0], [first], [n_q])
            out = torch.empty(n_q, Dv, device=dev)
            K().attention_general(q, out, kc, vc, table, page, b.token_seq, b.token_pos, b.seq_slot, n_heads=1,
                                  n_kv_heads=1, head_dim=D, window_kind=K().WINDOW_KINDS["sliding"], window_size=window,
                                  scale=1.0, value_dim=Dv, keep_first=keep)
            got = out[-1, 0].item()
            if seen:
                assert abs(got - (target + 1)) < 1e-3, (target, qpos, got)
            else:                                           # every visible key scores zero: the mean of their values
                vis = [p for p in range(qpos + 1) if P.visible(qpos, p, window, keep)]
                assert target not in vis and abs(got - sum(p + 1 for p in vis) / len(vis)) < 1e-2, (target, qpos, got)
        kc[pg, 0, off] = old


def _masked_reference(q, k, v, pos, window, keep, scale):
    """q [NH, D] at position pos; k, v [n, NKV, D]: softmax over the keys that `P.visible` lets through."""
    NH, G = q.shape[0], q.shape[0] // k.shape[1]
    vis = [j for j in range(pos + 1) if P.visible(pos, j, window, keep)]
    out = torch.empty(NH, v.shape[2], dtype=F64)
    for h in range(NH):
        sc = (k[vis, h // G].double() @ q[h].double()) * scale
        out[h] = torch.softmax(sc, 0) @ v[vis, h // G].double()
    return out


@pytest.mark.parametrize("NH,NKV,D,window,keep", [(8, 2, 128, 130, 70), (6, 6, 64, 64, 200), (4, 1, 64, 300, 1),
                                                  (4, 4, 128, 5, 128), (2, 1, 64, 129, 257)])
def test_kept_first_positions_in_the_tensor_core_kernels(NH, NKV, D, window, keep):
    """The decode kernel (one split and several) and the prefill kernel with kept first positions below a sliding
    window: sequences shorter than the kept range, with the kept range inside the window, next to it and hundreds of
    positions below it, kept ranges that end inside a page and inside a key tile, query tiles whose two halves'
    windows begin in different key tiles; the general kernel on the same inputs."""
    import test_gpu_kernels as TK
    page, scale = 64, 1.7 / math.sqrt(D)
    lengths = [1, 64, 65, 500, 129, 900, 258, 386]
    k, v, table = TK.paged_cache(len(lengths), lengths, NKV, D, page, torch.bfloat16, seed=3)
    T = len(lengths)
    q = TK.rnd(T, NH * D, dtype=torch.bfloat16, seed=4)
    token_seq = torch.arange(T, dtype=torch.int32, device="cuda")
    token_pos = torch.tensor([l - 1 for l in lengths], dtype=torch.int32, device="cuda")
    seq_slot = torch.arange(1, T + 1, dtype=torch.int32, device="cuda")
    kw = dict(n_heads=NH, n_kv_heads=NKV, head_dim=D, window_kind=K().WINDOW_KINDS["sliding"], window_size=window,
              scale=scale, keep_first=keep)
    refs = []
    for i, l in enumerate(lengths):
        kk, vv = TK.gather_kv(k, table, i + 1, l, page), TK.gather_kv(v, table, i + 1, l, page)
        refs.append(_masked_reference(q[i].float().view(NH, D).cpu(), kk.cpu(), vv.cpu(), l - 1, window, keep, scale).reshape(-1))
    outs = {"general": torch.empty_like(q)}
    K().attention_general(q, outs["general"], k, v, table, page, token_seq, token_pos, seq_slot, **kw)
    for splits in (1, 3, 7):
        outs[f"decode{splits}"] = torch.empty_like(q)
        K().attention_decode(q, outs[f"decode{splits}"], k, v, table, page, token_seq, token_pos, seq_slot,
                             n_splits=splits, **kw)
    torch.cuda.synchronize()
    for name, out in outs.items():
        for i in range(T):
            e = (out[i].double().cpu() - refs[i]).abs().max().item()
            assert e <= 1.5e-2 * max(1.0, refs[i].abs().max().item()), (name, i, lengths[i], e)
    c = TK._prefill_case(NH, NKV, D, ("sliding", window), [(0, 1), (0, 300), (70, 200), (100, 140), (400, 300), (0, 700),
                                                           (513, 256), (640, 130)], tile=256)
    out = torch.full_like(c["q"], float("nan"))
    K().attention_prefill(c["q"], out, c["k"], c["v"], c["table"], page, c["token_seq"], c["token_pos"], c["seq_slot"],
                          c["tile_tok0"], c["tile_rows"], **kw)
    torch.cuda.synchronize()
    assert int(K().tc_error_flag("cuda")[0]) == 0
    kk = [TK.gather_kv(torch.nan_to_num(c["k"]), c["table"], i + 1, l, page).cpu() for i, l in enumerate(c["lengths"])]
    vv = [TK.gather_kv(torch.nan_to_num(c["v"]), c["table"], i + 1, l, page).cpu() for i, l in enumerate(c["lengths"])]
    qc = c["q"].float().cpu()
    for t, (sq, pos) in enumerate(zip(c["seq"], c["pos"])):
        if t % 3 and pos % 64 not in (0, 1, 63) and pos not in (keep - 1, keep, keep + window - 1, keep + window):
            continue                                      # every third row, and every row at an edge
        ref = _masked_reference(qc[t].view(NH, D), kk[sq], vv[sq], pos, window, keep, scale).reshape(-1)
        e = (out[t].double().cpu() - ref).abs().max().item()
        assert e <= 1.5e-2 * max(1.0, ref.abs().max().item()), ("prefill", t, sq, pos, e)


def test_rotation_then_head_norm_in_the_preparation_kernel():
    g = torch.Generator().manual_seed(8)
    dev, T, H, G, D, Dv, dims, page = "cuda", 6, 3, 1, 20, 12, 8, 64
    rows = torch.randn(T, (H + G) * D + G * Dv, generator=g)
    f = torch.tensor([100.0 ** (-2.0 * i / dims) / 3.0 for i in range(dims // 2)])
    b = FakeBatch([0], [61], [T])                           # positions 61..66: the write crosses a page border
    table = torch.tensor([[3, 1]], dtype=torch.int32, device=dev)
    kc, vc = torch.zeros(4, G, page, D, device=dev), torch.zeros(4, G, page, Dv, device=dev)
    q = torch.empty(T, H * D, device=dev)
    K().qkv_prepare(rows.to(dev), q, kc, vc, table, page, b.token_seq, b.token_pos, b.seq_slot, n_heads=H, n_kv_heads=G,
                    head_dim=D, value_dim=Dv, norm_eps=1e-5, inv_freq=f.to(dev), rotary_dims=dims, head_norm=True)
    pos = torch.arange(61, 61 + T)
    want_q = P.rms_norm(P.rotate(rows[:, :H * D].double().view(T, H, D), pos, dims, 100.0, 3.0), None, 1e-5)
    want_k = P.rms_norm(P.rotate(rows[:, H * D:(H + G) * D].double().view(T, G, D), pos, dims, 100.0, 3.0), None, 1e-5)
    assert (q.cpu().double().view(T, H, D) - want_q).abs().max() < 1e-5
    for t in range(T):
        p = 61 + t
        pg = int(table[0, p // page])
        assert (kc[pg, 0, p % page].cpu().double() - want_k[t, 0]).abs().max() < 1e-5
        assert (vc[pg, 0, p % page].cpu() - rows[t, (H + G) * D:]).abs().max() == 0


# ---- the model -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_and_token_by_token(models, name, dtype):
    """A prompt in one step with logits everywhere, and the same tokens one by one from the first: both are the plain
    implementation's, which knows no cache."""
    b = models[name]
    toks = V.tokens(150, b.cfg["vocab"], 5)
    r = Run(b.engine(dtype))
    r.step([("whole", toks, range(len(toks)))])
    r.end("whole")
    for i, t in enumerate(toks[:90]):
        r.step([("single", [t], [0])])
    r.check(b, {"whole": toks, "single": toks}, TOL[dtype])


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_several_sizes(models, name):
    """A prompt cut into portions of 2, 3, 64, 1, 17, ... tokens, with cuts inside pages, windows and the kept first
    tokens; in float32 the logits are also those of the single step, to rounding."""
    b = models[name]
    toks = V.tokens(200, b.cfg["vocab"], 6)
    for dtype in ("float32", "bfloat16"):
        e = b.engine(dtype)
        r = Run(e)
        at = 0
        for n in (2, 3, 64, 1, 17, 2, 70, 5, 36):
            r.step([("p", toks[at:at + n], range(n))])
            at += n
        assert at == 200
        r.check(b, {"p": toks}, TOL[dtype])
        if dtype == "float32":
            one = Run(e)
            one.step([("w", toks, range(200))])
            d = err(torch.stack([r.logits["p"][i] for i in range(200)]), torch.stack([one.logits["w"][i] for i in range(200)]))
            assert d < 2e-5, d


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_batches_in_reused_slots(models, name, dtype):
    """Requests of 1 to 130 tokens start together, are decoded together, end at different steps; a second group then
    runs in the slots and pages the first gave back (two slots only).  Every logit is the request's own."""
    b = models[name]
    vocab = b.cfg["vocab"]
    reqs = {f"r{i}": V.tokens(n, vocab, 60 + i) for i, n in enumerate((1, 75, 130, 9, 66, 140))}
    e = b.engine(dtype, max_seqs=3, max_tokens=640)
    r = Run(e)
    for group in (("r0", "r1", "r2"), ("r3", "r4", "r5")):
        head = {i: max(1, len(reqs[i]) - 20) for i in group}
        r.step([(i, reqs[i][:head[i]], [head[i] - 1]) for i in group])
        live, k = [i for i in group if head[i] < len(reqs[i])], 0
        for i in group:
            if i not in live:
                r.end(i)
        while live:
            r.step([(i, [reqs[i][head[i] + k]], [0]) for i in live])
            k += 1
            for i in [i for i in live if head[i] + k == len(reqs[i])]:
                r.end(i)
                live.remove(i)
        e.cache.check_consistency()
    assert e.cache.free_slots == 3 and all(g.pages_held() == 0 for g in e.cache.groups)
    r.check(b, reqs, TOL[dtype])


@pytest.mark.parametrize("name", ["A", "B"])
def test_steps_larger_than_the_engine_takes_run_as_pieces(models, name):
    """An engine that takes 50 tokens a step gets steps of 191 and of 3 x 1 tokens: the first runs as pieces (whole
    sequences, then runs of a long one) against the cache and state the pieces before left; same logits."""
    b = models[name]
    vocab = b.cfg["vocab"]
    reqs = {"x": V.tokens(123, vocab, 80), "y": V.tokens(8, vocab, 81), "z": V.tokens(66, vocab, 82)}
    for dtype in ("float32", "bfloat16"):
        r = Run(b.engine(dtype, max_step_tokens=50, max_seqs=3, max_tokens=512))
        r.step([("x", reqs["x"][:120], range(0, 120, 7)), ("y", reqs["y"][:7], [0, 6]), ("z", reqs["z"][:64], [1, 49, 50, 63])])
        for k in range(1):
            r.step([("x", reqs["x"][120:121], [0]), ("y", reqs["y"][7:8], [0]), ("z", reqs["z"][64:65], [0])])
        r.end("y")
        r.step([("x", reqs["x"][121:123], [0, 1]), ("z", reqs["z"][65:66], [0])])
        r.check(b, reqs, TOL[dtype])


def test_heads_of_128_through_the_model(tmp_path):
    """Head size 128 on both sides (the 16-byte-per-lane preparation kernel, both tensor-core attention kernels with
    kept tokens that end inside a key tile and beyond one, a 256-row state): a prompt of 380 tokens and 40 decoded."""
    cfg = V.model([V.layer(V.left(4, 2, 128, 128, window=100, keep_first=70, rot_dims=128, factor=2.0), V.right(4, 2, 64, 128, 4), V.dense(512, 3.0)),
                   V.layer(V.left(8, 1, 128, 128, window=200, keep_first=130, rot_dims=128), V.right(2, 2, 128, 128, 3), V.moe(128, 8, 2, shared_ff=128)),
                   V.layer(V.left(2, 2, 128, 128, rot_dims=64), V.right(2, 1, 256, 64, 2), None)],
                  width=256, vocab=500, loop=(0, 2, 2), mult=0.5)
    b = Built(cfg, 77, tmp_path, ranks=(24, 24))
    toks = V.tokens(420, 500, 3)
    for dtype in ("float32", "bfloat16"):
        r = Run(b.engine(dtype, max_tokens=2048, max_seqs=2))
        r.step([("a", toks[:380], range(380))])
        for i in range(380, 420):
            r.step([("a", toks[i:i + 1], [0])])
        r.check(b, {"a": toks}, TOL[dtype])


def test_window_edges_and_kept_tokens_through_the_model(tmp_path):
    """One layer, one head, values that tell positions apart: moving the window or the kept count by one changes the
    logits as the plain implementation says, in a prompt and token by token, with the edge on a page border."""
    base = V.model([V.layer(V.left(1, 1, 16, 16, window=64, keep_first=64, rot_dims=16, scale=0.3),
                            V.right(1, 1, 8, 8, 2), None)], width=24, vocab=50, mult=1.0)
    toks = V.tokens(150, 50, 9)
    last = []
    for window, keep in ((64, 64), (63, 65), (65, 63), (1, 0), (128, 1)):
        cfg = copy.deepcopy(base)
        cfg["layers"][0]["mixer"]["left"]["mask"] = {"size": window, "keep_first": keep}
        b = Built(cfg, 31, tmp_path)
        r = Run(b.engine("float32"))
        r.step([("x", toks[:126], range(126))])
        for i in range(126, 150):
            r.step([("x", toks[i:i + 1], [0])])
        r.check(b, {"x": toks}, TOL["float32"])
        last.append(b.plain(toks)[-1])
    for i in range(1, len(last)):                           # the variants do differ where the edge moved
        assert (last[i] - last[0]).abs().max() > 1e-4, i


def test_a_far_token_among_hundreds_and_long_decoding(models):
    """700 tokens: the recurrent side carries the first tokens across many pages, the kept first tokens stay readable
    after their pages' neighbours were given back, and 120 tokens are decoded past several windows and a page border."""
    b = models["A"]
    toks = V.tokens(700, b.cfg["vocab"], 17)
    for dtype in ("float32", "bfloat16"):
        e = b.engine(dtype, max_tokens=1024, max_seqs=2)
        r = Run(e)
        r.step([("far", toks[:580], [0, 1, 300, 579])])
        held = max(g.pages_held() for g in e.cache.groups)
        for i in range(580, 700):
            r.step([("far", toks[i:i + 1], [0])])
        assert max(g.pages_held() for g in e.cache.groups) <= held       # windows give pages back, kept pages stay
        r.check(b, {"far": toks}, TOL[dtype])


def test_other_constants_change_the_result_as_the_plain_implementation_says(tmp_path):
    base = V.model([V.layer(V.left(2, 2, 16, 16, window=20, keep_first=4, rot_dims=8, factor=2.0), V.right(2, 2, 16, 16, 3),
                            V.dense(40, 1.0)),
                    V.layer(V.left(2, 1, 8, 24, window=6, rot_dims=8), V.right(4, 2, 8, 8, 2), V.moe(16, 4, 2, shared_ff=16))],
                   width=32, vocab=70, loop=(0, 1, 2), mult=0.5)
    changes = {
        "base": lambda c: None,
        "mult": lambda c: c.update(residual_mult=1.0), "no_mult_key": lambda c: c.pop("residual_mult"),
        "eps": lambda c: c["norm"].update(eps=1e-2), "no_loop": lambda c: c.pop("loop"),
        "loop_all": lambda c: c.update(loop={"start": 0, "stop": 2, "times": 2}),
        "factor": lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(factor=1.0),
        "no_scaling": lambda c: c["layers"][0]["mixer"]["left"]["rot"].pop("scaling"),
        "no_rot": lambda c: c["layers"][1]["mixer"]["left"].pop("rot"),
        "scale": lambda c: c["layers"][0]["mixer"]["left"].update(scale=0.9),
        "no_mask": lambda c: c["layers"][1]["mixer"]["left"].pop("mask"),
        "limit": lambda c: c["layers"][0]["mlp"].update(limit=0.25),
        "top": lambda c: c["layers"][1]["mlp"]["router"].update(top=4),
        "no_shared": lambda c: c["layers"][1]["mlp"].pop("shared"),
        "no_mlp": lambda c: c["layers"][0].update(mlp=None),
        "conv": lambda c: c["layers"][0]["mixer"]["right"].update(conv=5),
    }
    toks = V.tokens(40, 70, 2)
    seen = {}
    for key, change in changes.items():
        cfg = copy.deepcopy(base)
        change(cfg)
        b = Built(cfg, 21, tmp_path)
        r = Run(b.engine("float32"))
        r.step([("x", toks[:25], range(25))])
        for i in range(25, 40):
            r.step([("x", toks[i:i + 1], [0])])
        r.check(b, {"x": toks}, TOL["float32"])
        seen[key] = b.plain(toks)
    assert torch.equal(seen["mult"], seen["no_mult_key"]) and torch.equal(seen["factor"], seen["no_scaling"])
    for key in ("mult", "eps", "no_loop", "loop_all", "factor", "no_rot", "scale", "no_mask", "limit", "top", "no_shared",
                "no_mlp", "conv"):
        assert (seen[key] - seen["base"]).abs().max() > 1e-3, key


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_configurations_drawn_from_a_seed(seed, tmp_path):
    """Every size, option and constant drawn from a seed: a prompt with logits everywhere, a second request in a
    portion and then both decoded together, in float32 to rounding and in bfloat16."""
    import random
    cfg = V.draw_config(seed)
    rng = random.Random(seed)
    b = Built(cfg, 40 + seed, tmp_path, ranks=(rng.choice([1, 5, 24]), rng.choice([2, 8, 17])))
    vocab = cfg["vocab"]
    ta, tb = V.tokens(110, vocab, seed), V.tokens(75, vocab, seed + 100)
    for dtype in ("float32", "bfloat16"):
        r = Run(b.engine(dtype, max_tokens=1024, max_seqs=2))
        r.step([("a", ta[:90], range(90)), ("b", tb[:3], range(3))])
        r.step([("b", tb[3:70], range(67))])
        for i in range(5):
            r.step([("a", ta[90 + i:91 + i], [0]), ("b", tb[70 + i:71 + i], [0])])
        r.end("b")
        for i in range(95, 110):
            r.step([("a", ta[i:i + 1], [0])])
        r.check(b, {"a": ta, "b": tb}, TOL[dtype])


def test_layers_recorded_run_by_run(models):
    """The residual after every layer run (a looped layer counts each time) is the plain implementation's."""
    b = models["A"]
    toks = V.tokens(30, b.cfg["vocab"], 4)
    want = []
    P.forward(b.cfg, b.W, toks, want)
    e = b.engine("float32")
    e.model.layer_capture = []
    Run(e).step([("x", toks, [29])])
    assert len(e.model.layer_capture) == len(want) == 6
    for got, w in zip(e.model.layer_capture, want):
        assert (got.cpu().double() - w).abs().max() < 2e-4 * w.abs().max()


def test_greedy_generation_through_the_entry_point(models):
    """`Model.generate` (scheduler, sampler, decode graphs) picks the plain implementation's tokens: unequal prompts,
    more requests than slots."""
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


def test_random_weights_mode_and_command_line(models):
    """A folder drawn by the library's random mode loads and generates; bin/llama_infer knows the family by its
    config.json and its greedy tokens are the plain implementation's."""
    from cpi_b200.engine import Engine
    e = Engine.from_random(V.MIXED_B, seed=3, dtype="bfloat16", max_tokens=512)
    out = Run(e)
    out.step([("x", V.tokens(70, 384, 1), [69])])
    assert torch.isfinite(out.logits["x"][69]).all()
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
    assert "Savenex" in r.stdout and "scan" in r.stdout


def test_replay_tool_runs_a_savenex_folder(models, tmp_path):
    """bin/trace_run in a process of its own: a request whole, and two requests batched then decoded."""
    import numpy as np
    b = models["B"]
    vocab = b.cfg["vocab"]
    ta, tb = V.tokens(80, vocab, 40), V.tokens(21, vocab, 41)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ta, "want": list(range(80))}], "end": ["a"]},
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
        rd = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, vocab).copy())
        ra, rb = b.plain(ta), b.plain(tb)
        got = torch.cat([rd(i) for i in range(4)])
        want = torch.cat([ra, torch.stack([ra[69], rb[20], ra[70], ra[71]])])
        assert got.shape == want.shape and err(got, want, dtype == "bfloat16") < TOL[dtype]
