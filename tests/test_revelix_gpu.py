"""Revelix on the GPU against the plain implementation: each mechanism's kernels alone, then whole models in float32
and bfloat16 - whole prompts, token-by-token decoding, portions down to two tokens, unequal batches against each
request alone, slots and pages used again, keys far away, at page borders, at the window's edges and at the edge of the
kept first positions, long decoding, greedy generation through the engine's entry point and scheduler, the command line
and the trace runner."""

import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch
import torch.nn.functional as F

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200 import kernels as K
from flashdecode_cuda_b200.parts.rope import RotaryScaled
from helpers import prompts_for, rel_err
from revelix_helpers import (MODEL_TOL as TOL, REVELIX, Truth, oracle_logits, plain_greedy, random_config, raw_config, truth,
                             weights_of, write_folder)
from plain import revelix_plain as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda"
NAMES = ["P", "Q", "R"]
DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KTOL = {"float32": 2e-5, "bfloat16": 2e-2}


class _Rt:
    device = torch.device(DEV)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def step_arrays(ctx_lens, q_lens, slots):
    """Index arrays of a step whose rows bring q_lens[i] tokens after ctx_lens[i] cached ones."""
    tok_row, tok_pos, starts = [], [], []
    for r, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        starts.append(len(tok_row))
        tok_row += [r] * n
        tok_pos += list(range(c, c + n))
    return i32(tok_row), i32(tok_pos), i32(slots), i32(starts), i32(q_lens), i32(ctx_lens)


def new_status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(1, 64), (5, 100), (37, 1027), (3, 4096 + 8)])
def test_dynamic_tanh_with_the_deferred_add(dtype, T, H):
    torch.manual_seed(T + H)
    resid = torch.randn(T, H) * 2
    delta = torch.randn(T, H).to(TD[dtype])
    w, b, alpha = 1 + 0.1 * torch.randn(H), 0.1 * torch.randn(H), 0.37
    r = resid.to(DEV)
    out = torch.zeros(T, H, dtype=TD[dtype], device=DEV)
    K.add_dyn_tanh(delta.to(DEV), r, w.to(DEV), b.to(DEV), alpha, out)
    total = resid.double() + delta.double()
    assert rel_err(r, total) < 1e-6                                  # the stream keeps the sum in float32
    assert rel_err(out, P.dyn_tanh(total, w.double(), b.double(), torch.tensor(alpha).double())) < KTOL[dtype]
    rows = i32([T - 1, 0])                                           # the final norm: gathered rows, nothing written back
    before = r.clone()
    out2 = torch.zeros(2, H, dtype=TD[dtype], device=DEV)
    K.add_dyn_tanh(None, r, w.to(DEV), b.to(DEV), alpha, out2, rows=rows, write_resid=False)
    assert torch.equal(r, before) and torch.equal(out2, out[[T - 1, 0]])


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_branch_activation(dtype):
    z = torch.cat([torch.linspace(-30, 30, 2001), torch.tensor([0.0, -0.0, 1e-6, -1e-6, -100.0])]).to(TD[dtype])
    for p, q in ((0.3, -0.7), (-25.0, 25.0), (2.0, 0.0)):                # softplus far on both sides of its threshold
        pq = torch.tensor([p, q])
        out = torch.zeros_like(z, device=DEV)
        K.quad_exp_act(z.to(DEV), pq.to(DEV), out)
        want = P.two_branch_act(z.double(), pq[0].double(), pq[1].double())
        err = (out.double().cpu() - want).abs() / (1 + want.abs())
        assert float(err.max()) < (1e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dims,base,scaling", [(16, 10000.0, None), (48, 1e6, (8.0, 1024, 32.0, 1.0)),
                                               (2, 100.0, (4.0, 64, 16.0, 2.0)), (64, 500.0, (32.0, 16, 4.0, 0.5)),
                                               (8, 10000.0, (2.0, 4096, 1.0, 1.0))])     # fast == slow: a step, not a ramp
def test_rotation_tables_follow_the_stretched_frequencies(dims, base, scaling):
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    pos = RotaryScaled(dims, base, sc)
    pos.prepare(300, _Rt)
    f, mag = P.rot_frequencies(dims, base, sc)
    a = torch.outer(torch.arange(300).double(), f)
    assert pos.cos.shape[1] == dims // 2 and pos.cos.shape[0] >= 300
    assert float((pos.cos[:300].cpu().double() - a.cos() * mag).abs().max()) < 2e-7 * max(mag, 1)
    assert float((pos.sin[:300].cpu().double() - a.sin() * mag).abs().max()) < 2e-7 * max(mag, 1)
    if sc:
        plain, _ = P.rot_frequencies(dims, base, None)
        assert bool((f <= plain + 1e-18).all()) and bool((f >= plain / sc["factor"] - 1e-18).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,rot,d,dv,cuts", [(3, 8, 16, 32, [5, 1, 1, 6]), (4, 16, 16, 16, [2, 2, 9]),
                                                (1, 0, 32, 16, [7, 1]), (2, 32, 32, 48, [1, 1, 1, 10]),
                                                (5, 6, 8, 8, [3, 1, 1, 10, 1])])
def test_convolution_interleaved_rotation_and_append(dtype, taps, rot, d, dv, cuts):
    """Two sequences fed in portions (some of one token, some shorter than the taps), their channels starting at a
    column offset of a wider projection: q, the cached keys and values and the carried state equal the plain
    convolution and the plain rotation of pairs (2i, 2i + 1) with stretched frequencies over the whole sequences."""
    torch.manual_seed(taps * 100 + rot)
    dt = TD[dtype]
    n_q, n_kv, bs, col0 = 3, 1, 4, 10
    C = (n_q + n_kv) * d + n_kv * dv
    S = sum(cuts)
    lens = [S, S - 3]
    u = [torch.randn(n, col0 + C + 6).to(dt) for n in lens]          # columns before and after that the kernel must leave alone
    w = torch.randn(C, taps) * 0.5
    k_pool = torch.zeros(16, n_kv, bs, d, dtype=dt, device=DEV)
    v_pool = torch.zeros(16, n_kv, bs, dv, dtype=dt, device=DEV)
    table = torch.full((4, 8), -1, dtype=torch.int32, device=DEV)
    slots = [2, 0]
    table[2, :4] = i32([5, 1, 7, 3])
    table[0, :4] = i32([0, 9, 2, 11])
    state = torch.zeros(4, max(taps - 1, 1), C, device=DEV) if taps > 1 else None
    sc = {"factor": 4.0, "original": 16, "fast": 2.0, "slow": 0.5}
    pos = RotaryScaled(rot, 100.0, sc) if rot else None
    if pos:
        pos.prepare(64, _Rt)
    status = new_status()
    q_got = [torch.zeros(n, n_q * d) for n in lens]
    done = [0, 0]
    for cut in cuts:
        rows = [r for r in range(2) if done[r] < lens[r]]
        q_lens = [min(cut, lens[r] - done[r]) for r in rows]
        proj = torch.cat([u[r][done[r]:done[r] + n] for r, n in zip(rows, q_lens)]).to(DEV).contiguous()
        tok_row, tok_pos, row_slot, q_start, q_len, _ = step_arrays([done[r] for r in rows], q_lens, [slots[r] for r in rows])
        q_out = torch.zeros(proj.shape[0], n_q * d, dtype=dt, device=DEV)
        single = max(q_lens) == 1
        K.conv_rope_append(proj, w.to(DEV), state, q_out, pos.cos if rot else None, pos.sin if rot else None, rot, tok_row,
                           tok_pos, row_slot, q_start, q_len, k_pool, v_pool, table, n_q, n_kv, d, dv, True, single, status,
                           interleaved=True, first_col=col0)
        if state is not None and not single:
            K.conv_state_update(proj, state, row_slot, q_start, q_len, len(rows), first_col=col0)
        at = 0
        for r, n in zip(rows, q_lens):
            q_got[r][done[r]:done[r] + n] = q_out[at:at + n].float().cpu()
            at += n
            done[r] += n
    assert int(status.item()) == 0
    fr, mag = P.rot_frequencies(rot, 100.0, sc) if rot else (None, 1.0)
    for r in range(2):
        n = lens[r]
        x = u[r][:, col0:col0 + C].double()
        y = P.short_conv(x, w.double())
        q_want = y[:, :n_q * d].reshape(n, n_q, d)
        k_want = y[:, n_q * d:(n_q + n_kv) * d].reshape(n, n_kv, d)
        if rot:
            q_want = P.rotate(q_want, torch.arange(n), rot, fr, mag, interleaved=True)
            k_want = P.rotate(k_want, torch.arange(n), rot, fr, mag, interleaved=True)
        v_want = y[:, (n_q + n_kv) * d:].reshape(n, n_kv, dv)
        assert rel_err(q_got[r], q_want.reshape(n, -1)) < KTOL[dtype]
        blocks = table[slots[r]].tolist()
        k_got = torch.stack([k_pool[blocks[p // bs], :, p % bs] for p in range(n)]).float().cpu()
        v_got = torch.stack([v_pool[blocks[p // bs], :, p % bs] for p in range(n)]).float().cpu()
        assert rel_err(k_got, k_want) < KTOL[dtype] and rel_err(v_got, v_want) < KTOL[dtype]
        if state is not None:
            assert torch.equal(state[slots[r]].cpu(), u[r][n - (taps - 1):, col0:col0 + C].float())


def _scan_in_portions(dt, proj_of, cols, mode, H, d, dv, lens, cuts, segments=False, **kw):
    """Run ``K.linear_scan`` over two sequences cut into portions; returns (outputs per sequence, final states).
    ``segments``: with scratch memory, so that portions longer than two segments run as segments side by side."""
    slots = [3, 1]
    state = torch.zeros(5, H, d, dv, device=DEV)
    state[4] = 7.0                                           # a slot nobody uses stays as it is
    status = new_status()
    got = [torch.zeros(n, H * dv) for n in lens]
    done = [0, 0]
    for cut in cuts:
        rows = [r for r in range(2) if done[r] < lens[r]]
        if not rows:
            break
        q_lens = [min(cut, lens[r] - done[r]) for r in rows]
        proj = torch.cat([proj_of[r][done[r]:done[r] + n] for r, n in zip(rows, q_lens)]).to(dt).to(DEV).contiguous()
        _, _, row_slot, q_start, q_len, ctx_len = step_arrays([done[r] for r in rows], q_lens, [slots[r] for r in rows])
        out = torch.full((proj.shape[0], H * dv), float("nan"), device=DEV)
        if segments:
            n_scr = K.linear_scan_scratch_floats(proj.shape[0], len(rows), H, d, dv)
            kw = dict(kw, max_q_len=max(q_lens), scratch=torch.full((n_scr,), float("nan"), device=DEV))
        K.linear_scan(proj, cols[0], cols[1], cols[2], state, out, mode, row_slot, q_start, q_len, ctx_len, len(rows),
                      H, d, dv, True, status, **kw)
        at = 0
        for r, n in zip(rows, q_lens):
            got[r][done[r]:done[r] + n] = out[at:at + n].cpu()
            at += n
            done[r] += n
    assert done == lens and int(status.item()) == 0
    assert bool((state[4] == 7.0).all())
    return got, [state[s].cpu() for s in slots]


SCAN_CASES = [  # heads, d, dv, rotated dims
    (2, 16, 8, 16), (3, 24, 40, 8), (1, 64, 64, 0), (2, 136, 24, 136), (1, 12, 6, 4), (4, 128, 128, 64), (1, 256, 72, 2)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv,rot", SCAN_CASES)
def test_retention_recurrence_in_portions(dtype, H, d, dv, rot):
    """S_t = g S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with rotated q and k, from portions of many sizes, against the plain
    token-by-token recurrence over the whole sequences.  Decays include 1 (nothing is forgotten) and 0.5."""
    torch.manual_seed(H * d + dv)
    dt = TD[dtype]
    lens = [90, 41]
    nk, nv, extra = H * d, H * dv, 5
    proj_of = [(torch.randn(n, extra + 2 * nk + nv + 3)).to(dt).float() for n in lens]
    decay = ([1.0, 0.5, 0.97, 0.999] * H)[:H]
    pos = RotaryScaled(rot, 1000.0) if rot else None
    if pos:
        pos.prepare(128, _Rt)
    got, states = _scan_in_portions(dt, proj_of, (extra, extra + nk, extra + 2 * nk), K.SCAN_DECAY, H, d, dv, lens,
                                    [17, 1, 1, 2, 30, 3, 1, 16, 64], decay=torch.tensor(decay, device=DEV),
                                    cos=pos.cos if rot else None, sin=pos.sin if rot else None, rot_dims=rot, k_scale=d ** -0.5)
    for r, n in enumerate(lens):
        x = proj_of[r].double()
        q, k = x[:, extra:extra + nk].reshape(n, H, d), x[:, extra + nk:extra + 2 * nk].reshape(n, H, d)
        v = x[:, extra + 2 * nk:extra + 2 * nk + nv].reshape(n, H, dv)
        if rot:
            fr, mag = P.rot_frequencies(rot, 1000.0)
            q = P.rotate(q, torch.arange(n), rot, fr, mag, interleaved=False)
            k = P.rotate(k, torch.arange(n), rot, fr, mag, interleaved=False)
        want = P.decayed_recurrence(q, k * d ** -0.5, v, decay).reshape(n, nv)
        assert rel_err(got[r], want) < 2e-5                  # the recurrence itself is float32 in both dtypes
        final = torch.zeros(H, d, dv, dtype=torch.float64)
        for t in range(n):
            final = torch.tensor(decay).double()[:, None, None] * final + (k[t] * d ** -0.5)[:, :, None] * v[t][:, None, :]
        assert rel_err(states[r], final) < 2e-5


SEGMENT_CASES = [(2, 16, 8, 16), (3, 24, 40, 8), (2, 136, 24, 136), (2, 128, 128, 64), (1, 256, 72, 2)]
# portions that are many segments, exactly whole segments, one token more and less than that, two segments and one
# token (the shortest that is cut), and short ones that are not cut, each going on from the state the one before left
SEGMENT_LENS, SEGMENT_CUTS = [459, 262], [192, 129, 1, 63, 65, 3, 128]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv,rot", SEGMENT_CASES)
def test_retention_recurrence_in_segments(dtype, H, d, dv, rot):
    """Long portions run as segments side by side that are chained afterwards; against the plain token-by-token
    recurrence over the whole sequences, with two sequences of unequal length in every step."""
    assert K.linear_scan_segment() == 64
    torch.manual_seed(H * d + dv + 2)
    dt = TD[dtype]
    lens = SEGMENT_LENS
    nk, nv = H * d, H * dv
    proj_of = [(torch.randn(n, 2 * nk + nv + 3)).to(dt).float() for n in lens]
    decay = ([0.97, 1.0, 0.5, 0.999] * H)[:H]
    pos = RotaryScaled(rot, 1000.0)
    pos.prepare(512, _Rt)
    got, states = _scan_in_portions(dt, proj_of, (0, nk, 2 * nk), K.SCAN_DECAY, H, d, dv, lens, SEGMENT_CUTS, segments=True,
                                    decay=torch.tensor(decay, device=DEV), cos=pos.cos, sin=pos.sin, rot_dims=rot,
                                    k_scale=d ** -0.5)
    fr, mag = P.rot_frequencies(rot, 1000.0)
    for r, n in enumerate(lens):
        x = proj_of[r].double()
        q = P.rotate(x[:, :nk].reshape(n, H, d), torch.arange(n), rot, fr, mag, interleaved=False)
        k = P.rotate(x[:, nk:2 * nk].reshape(n, H, d), torch.arange(n), rot, fr, mag, interleaved=False) * d ** -0.5
        v = x[:, 2 * nk:2 * nk + nv].reshape(n, H, dv)
        assert rel_err(got[r], P.decayed_recurrence(q, k, v, decay).reshape(n, nv)) < 2e-5
        final = torch.zeros(H, d, dv, dtype=torch.float64)
        for t in range(n):
            final = torch.tensor(decay).double()[:, None, None] * final + k[t][:, :, None] * v[t][:, None, :]
        assert rel_err(states[r], final) < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv,rot", SEGMENT_CASES)
def test_gated_recurrence_in_segments(dtype, H, d, dv, rot):
    """The same with a forget gate per channel, whose product over a segment is what chains it to the next; lower bounds
    of 0 and 1 included, and gates near 0, whose products over a segment vanish."""
    torch.manual_seed(H * d + dv + 3)
    dt = TD[dtype]
    lens = SEGMENT_LENS
    nk, nv = H * d, H * dv
    proj_of = [(torch.randn(n, 2 * nk + nv) * 2).to(dt).float() for n in lens]
    for x in proj_of:
        x[:, nk + 1] -= 12.0                                 # a channel whose gate stays near its lower bound of 0
    lower = torch.rand(nk)
    lower[0], lower[1], lower[-1] = 0.0, 0.0, 1.0
    got, states = _scan_in_portions(dt, proj_of, (0, nk, 2 * nk), K.SCAN_GATED, H, d, dv, lens, SEGMENT_CUTS, segments=True,
                                    lower=lower.to(DEV))
    for r, n in enumerate(lens):
        x = proj_of[r].double()
        q = F.silu(x[:, :nk]).reshape(n, H, d)
        f = (lower.double() + (1 - lower.double()) * torch.sigmoid(x[:, nk:2 * nk])).reshape(n, H, d)
        v = x[:, 2 * nk:].reshape(n, H, dv)
        assert rel_err(got[r], P.gated_recurrence(q, f, v).reshape(n, nv)) < 2e-5
    assert bool((states[0][-1, -1] == 0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,d,dv,rot", SCAN_CASES)
def test_gated_recurrence_in_portions(dtype, H, d, dv, rot):
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T read by silu(q_t), f = lower + (1 - lower) sigmoid(z); lower bounds of
    0 and 1 included (a channel that forgets everything it may, and one that never changes)."""
    torch.manual_seed(H * d + dv + 1)
    dt = TD[dtype]
    lens = [70, 33]
    nk, nv = H * d, H * dv
    proj_of = [(torch.randn(n, 2 * nk + nv) * 2).to(dt).float() for n in lens]
    lower = torch.rand(nk)
    lower[0], lower[-1] = 0.0, 1.0
    got, states = _scan_in_portions(dt, proj_of, (0, nk, 2 * nk), K.SCAN_GATED, H, d, dv, lens, [2, 2, 19, 1, 1, 1, 40, 5],
                                    lower=lower.to(DEV))
    for r, n in enumerate(lens):
        x = proj_of[r].double()
        q = F.silu(x[:, :nk]).reshape(n, H, d)
        f = (lower.double() + (1 - lower.double()) * torch.sigmoid(x[:, nk:2 * nk])).reshape(n, H, d)
        v = x[:, 2 * nk:].reshape(n, H, dv)
        assert rel_err(got[r], P.gated_recurrence(q, f, v).reshape(n, nv)) < 2e-5
    assert bool((states[0][-1, -1] == 0).all())              # the channel whose gate is 1 never took anything in


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dv,weighted,gated", [(3, 40, False, True), (2, 8, True, False), (1, 72, True, True), (5, 6, False, False)])
def test_norm_per_head_with_gate_into_a_shared_buffer(dtype, H, dv, weighted, gated):
    torch.manual_seed(H + dv)
    dt = TD[dtype]
    T, eps, scale, col, gcol = 9, 1e-3, 1.3, 4, 2
    o = torch.randn(T, H * dv) * 0.05                                  # small outputs: eps matters
    w = torch.randn(dv) if weighted else None
    gate = torch.randn(T, gcol + H * dv + 1).to(dt) if gated else None
    out = torch.full((T, col + H * dv + 3), 9.0, dtype=dt, device=DEV)
    K.head_norm_gate(o.to(DEV), out, col, H, dv, eps, w.to(DEV) if weighted else None,
                     gate.to(DEV) if gated else None, gcol, scale)
    want = P.unit_rms(o.double().view(T, H, dv), eps)
    if weighted:
        want = want * w.double()
    want = want.reshape(T, H * dv) * scale
    if gated:
        want = want * F.silu(gate[:, gcol:gcol + H * dv].double())
    assert rel_err(out[:, col:col + H * dv], want) < KTOL[dtype]
    assert bool((out[:, :col] == 9.0).all()) and bool((out[:, col + H * dv:] == 9.0).all())


def _mixed_attention_case(dtype, d, dv, G, n_kv, window, keep, softcap, bs, S, portions, seed, far=False, tensor_cores=True):
    """Keys that stand out: every seventh position (each is the oldest key inside the window of one query and the
    newest outside it for the next), the last kept position and the first that is not kept, and - with ``far`` - one
    key hundreds of positions back that only the kept range or a long window still shows.  A visibility that is one
    position off, a sink left out or heads mixed the wrong way changes the result by the size of a value."""
    torch.manual_seed(seed)
    dt = TD[dtype]
    n_q = G * n_kv
    q = torch.randn(S, n_q, d) * 0.3
    k = torch.randn(S, n_kv, d) * 0.3
    v = torch.randn(S, n_kv, dv)
    e = torch.zeros(d)
    e[3 % d] = 1.0
    marked = {p for p in range(S) if p % 7 == 0} | {keep - 1, keep} | ({2} if far else set())
    for p in marked:
        if 0 <= p < S:
            k[p] += 6.0 * e
    q += 2.0 * e
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    scale = 0.7
    sink = torch.randn(n_q) * 2
    talk = torch.eye(n_q) + 0.4 * torch.randn(n_q, n_q)
    want = P.mixed_head_attention(q.double(), k.double(), v.double(), scale, softcap, window, keep, sink.double(),
                                  talk.double()).reshape(S, n_q * dv)
    n_cols = -(-S // bs)
    k_pool = torch.zeros(n_cols + 3, n_kv, bs, d, dtype=dt, device=DEV)
    v_pool = torch.zeros(n_cols + 3, n_kv, bs, dv, dtype=dt, device=DEV)
    perm = torch.randperm(n_cols + 3)[:n_cols]
    table = torch.full((2, n_cols), -1, dtype=torch.int32, device=DEV)
    table[1] = perm.to(torch.int32).to(DEV)
    for p in range(S):
        k_pool[perm[p // bs], :, p % bs] = k[p].to(DEV)
        v_pool[perm[p // bs], :, p % bs] = v[p].to(DEV)
    status = new_status()
    got = torch.zeros(S, n_q * dv)
    at = 0
    for n in portions:
        n = min(n, S - at)
        if n <= 0:
            break
        tok_row, _, row_slot, q_start, q_len, ctx_len = step_arrays([at], [n], [1])
        n_splits, split_len, scratch = 1, 0, None
        if n == 1 and at + 1 > 64:
            split_len = 64
            n_splits = -(-(at + 1) // split_len)
            scratch = torch.zeros(K.attention_scratch_floats(1, n_q * n_kv, dv, n_splits), device=DEV)
        per_head = torch.full((n, n_q * n_kv * dv), float("nan"), device=DEV)
        K.attention_ext(q[at:at + n].reshape(n, n_q * d).to(DEV).contiguous(), k_pool, v_pool, per_head, table, tok_row,
                        row_slot, q_start, q_len, ctx_len, 1, n, n_q, n_kv, d, scale, window or 0, n_splits, split_len,
                        scratch, status, softcap=softcap or 0.0, keep_first=keep if window else 0, sink=sink.to(DEV),
                        all_value_heads=True, tensor_cores=tensor_cores)
        out = torch.full((n, 2 + n_q * dv), 5.0, dtype=dt, device=DEV)
        K.attn_head_mix(per_head, talk.to(DEV), out, 2, n_q, n_kv, dv, 1.0)
        assert bool((out[:, :2] == 5.0).all())
        got[at:at + n] = out[:, 2:].float().cpu()
        at += n
    assert at == S and int(status.item()) == 0
    err = (got.double() - want).abs().max(dim=1).values / want.abs().max()
    assert float(err.max()) < KTOL[dtype], (f"first wrong position {int((err >= KTOL[dtype]).nonzero()[0])} "
                                            f"(window {window}, {keep} kept)")


MIX_CASES = [  # d, dv, G, n_kv, window, kept, soft cap, block size, length
    (64, 64, 2, 2, 24, 5, 10.0, 16, 150),      # window edges inside pages
    (64, 64, 4, 1, 64, 0, None, 64, 200),      # a window of exactly one page, nothing kept, no cap
    (32, 48, 3, 2, 27, 30, 8.0, 8, 120),       # more kept positions than the window is long
    (48, 16, 1, 3, 9, 14, 30.0, 4, 100),       # one query head per key head: only the mixing joins heads
    (24, 40, 2, 2, None, 0, 2.0, 16, 90),      # no window: every earlier key
    (128, 128, 2, 1, 1, 1, 5.0, 32, 80),       # a window of the query itself, plus the very first key
    (8, 8, 2, 2, 40, 3, 20.0, 16, 330),        # keys far back: the kept ones stay visible 300 positions on
    (64, 64, 2, 2, 70, 5, 15.0, 16, 400),      # tiles of keys between the kept ones and the window that nobody sees
    (128, 128, 2, 2, 100, 70, 10.0, 64, 450),  # kept positions that fill more than one tile of keys
    (64, 64, 4, 2, 200, 130, None, 8, 500),    # kept positions that end inside the tile where a window starts
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", MIX_CASES)
@pytest.mark.parametrize("tensor_cores", [True, False])
def test_capped_windowed_attention_with_sink_and_mixed_heads_whole_prompt(dtype, case, tensor_cores):
    """With and without the tensor-core form of the kernel, which takes bfloat16 prompts with heads of 64 and 128."""
    d, dv, G, n_kv, window, keep, cap, bs, S = case
    _mixed_attention_case(dtype, d, dv, G, n_kv, window, keep, cap, bs, S, [S], seed=1, far=True, tensor_cores=tensor_cores)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", MIX_CASES)
def test_capped_windowed_attention_in_portions_and_token_by_token(dtype, case):
    d, dv, G, n_kv, window, keep, cap, bs, S = case
    w = window or 20
    _mixed_attention_case(dtype, d, dv, G, n_kv, window, keep, cap, bs, S, [w * 2 - 1, 2, w, 3, 129, 2] + [1] * S, seed=2,
                          far=True)
    _mixed_attention_case(dtype, d, dv, G, n_kv, window, keep, cap, bs, min(S, 3 * w + keep + 2), [1] * S, seed=3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,dv,T", [(6, 2, 24, 5), (4, 4, 8, 3), (32, 8, 64, 70), (64, 8, 256, 3), (5, 1, 40, 9)])
def test_heads_mixed_on_their_own_value_head(dtype, n_q, n_kv, dv, T):
    """out[t, h] = scale * sum_g mix[h, g] o[t, g, h's value head]; sizes whose rows fit shared memory and one that does not."""
    torch.manual_seed(n_q + dv)
    o = torch.randn(T, n_q, n_kv, dv)
    mix = torch.randn(n_q, n_q)
    out = torch.full((T, 3 + n_q * dv), 4.0, dtype=TD[dtype], device=DEV)
    K.attn_head_mix(o.reshape(T, -1).to(DEV), mix.to(DEV), out, 3, n_q, n_kv, dv, 0.7)
    G = n_q // n_kv
    want = torch.stack([0.7 * torch.einsum("g,tgj->tj", mix[h].double(), o[:, :, h // G].double()) for h in range(n_q)], dim=1)
    assert rel_err(out[:, 3:], want.reshape(T, n_q * dv)) < KTOL[dtype]
    assert bool((out[:, :3] == 4.0).all())


def test_sink_takes_its_share_and_nothing_else():
    """One query, one key: the weight of the key is e^s / (e^s + e^sink), so the output is that share of the value;
    with mixing weights of zero off the diagonal a head's output depends on its own sink only."""
    d = dv = 8
    n_q = n_kv = 2
    q = torch.zeros(1, n_q * d, device=DEV)
    k_pool = torch.zeros(1, n_kv, 4, d, device=DEV)
    v_pool = torch.ones(1, n_kv, 4, dv, device=DEV)
    table = i32([[0]])
    sink = torch.tensor([0.0, math.log(3.0)], device=DEV)
    tok_row, _, row_slot, q_start, q_len, ctx_len = step_arrays([0], [1], [0])
    per_head = torch.zeros(1, n_q * n_kv * dv, device=DEV)
    status = new_status()
    K.attention_ext(q, k_pool, v_pool, per_head, table, tok_row, row_slot, q_start, q_len, ctx_len, 1, 1, n_q, n_kv, d, 1.0,
                    0, 1, 0, None, status, sink=sink, all_value_heads=True)
    out = torch.zeros(1, n_q * dv, device=DEV)
    K.attn_head_mix(per_head, torch.eye(n_q, device=DEV), out, 0, n_q, n_kv, dv, 2.0)
    assert torch.allclose(out[0, :dv].cpu(), torch.full((dv,), 2.0 * 0.5), atol=1e-6)       # e^0 / (e^0 + e^0)
    assert torch.allclose(out[0, dv:].cpu(), torch.full((dv,), 2.0 * 0.25), atol=1e-6)      # e^0 / (e^0 + 3)


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("revelix")
    return {n: write_folder(tmp, n, seed=31) for n in NAMES}


@pytest.fixture(scope="module")
def engines(folders):
    return {(n, d): fd.load(folders[n], device="cuda", dtype=d) for n in NAMES for d in DTYPES}


def _vocab(name):
    return REVELIX[name]["vocab"]


def _lengths(name):
    # around the window (27 / 16 / 9), the kept positions (5 / 0 / 14), the taps and the pages
    return {"P": [1, 2, 5, 6, 27, 28, 33, 75, 140], "Q": [1, 16, 17, 64, 65, 129], "R": [3, 9, 10, 14, 15, 24, 100, 201]}[name]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("block_size", [8, 64])
def test_whole_prompts(engines, folders, name, dtype, block_size):
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=320, block_size=block_size)
    for p in prompts_for(_vocab(name), _lengths(name), seed=1):
        slot = cache.admit()
        got = eng.model.step(cache, [slot], [p], "all")
        assert truth(folders[name], p).excess(got, range(len(p)), dtype) < 1, f"prompt of {len(p)} tokens"
        cache.release(slot)
    eng.model.check_status()
    cache.check_invariants()


def test_every_layer_in_float32(engines, folders):
    """The residual stream after every layer against the plain one."""
    for name in NAMES:
        eng = engines[(name, "float32")]
        (p,) = prompts_for(_vocab(name), [45], seed=2)
        trace = []
        P.forward(raw_config(folders[name]), weights_of(folders[name]), p, trace=trace)
        cache = eng.model.new_cache(max_tokens=64)
        slot = cache.admit()
        eng.model.trace = {}
        eng.model.step(cache, [slot], [p], None)
        got, eng.model.trace = eng.model.trace, None
        assert len(trace) == len(eng.model.schedule)
        for i, want in enumerate(trace):
            assert rel_err(got[f"layer.{i}"], want) < 1e-5, f"{name}: layer {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_token_by_token_across_window_edges(engines, folders, name, dtype):
    """A prompt of one token or of thirty, then so many single tokens that every window of the model passes over
    decoded tokens and the kept positions are left behind while decoding."""
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=256, block_size=16)
    n_decode = {"P": 70, "Q": 45, "R": 50}[name]
    for head in (1, 30):
        (p,) = prompts_for(_vocab(name), [head + n_decode], seed=3 + head)
        want = truth(folders[name], p)
        slot = cache.admit()
        got = eng.model.step(cache, [slot], [p[:head]], "last")
        assert want.excess(got, [head - 1], dtype) < 1
        for i in range(head, len(p)):
            got = eng.model.step(cache, [slot], [[p[i]]], "last")
            assert want.excess(got, [i], dtype) < 1, f"position {i} of a request decoded from {head}"
        cache.release(slot)
    eng.model.check_status()
    cache.check_invariants()


def test_long_decoding_in_float32(engines, folders):
    """Four hundred single tokens after a short prompt: the states keep what the plain recurrences keep, and the
    window's pages are given back and used again."""
    name = "P"
    eng = engines[(name, "float32")]
    (p,) = prompts_for(_vocab(name), [420], seed=9)
    want = oracle_logits(folders[name], p)
    cache = eng.model.new_cache(max_tokens=512, block_size=8)
    slot = cache.admit()
    eng.model.step(cache, [slot], [p[:20]], None)
    for i in range(20, len(p)):
        got = eng.model.step(cache, [slot], [[p[i]]], "last")
        if i % 50 == 0 or i > 410:
            assert rel_err(got[0], want[i]) < TOL["float32"], f"position {i}"
    cache.release(slot)
    eng.model.check_status()
    cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_several_sizes(engines, folders, name, dtype):
    """A prompt cut into portions of 2, 3, 1, 7, 33, ... tokens gives the logits of the whole prompt."""
    eng = engines[(name, dtype)]
    (p,) = prompts_for(_vocab(name), [150], seed=5)
    want = truth(folders[name], p)
    cache = eng.model.new_cache(max_tokens=256, block_size=8)
    slot = cache.admit()
    whole = eng.model.step(cache, [slot], [p], "all").clone()
    cache.release(slot)
    for sizes in ([2] * 75, [3, 1, 7, 33, 2, 64, 5, 1, 1, 30, 3], [149, 1], [1, 149]):
        slot = cache.admit()
        at, rows = 0, []
        for n in sizes:
            rows.append(eng.model.step(cache, [slot], [p[at:at + n]], "all").clone())
            at += n
        assert at == len(p)
        got = torch.cat(rows)
        cache.release(slot)
        assert want.excess(got, range(len(p)), dtype) < 1
        apart = (got.double().cpu() - whole.double().cpu()).abs().amax(-1) / want.scale
        bound = want.allowed(dtype) if dtype == "bfloat16" else want.allowed(dtype) * 0.05
        assert bool((apart < bound).all()), f"portions {sizes[:4]}..."
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batch_equals_each_request_alone_and_slots_are_used_again(engines, folders, name, dtype):
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=64 * 8, block_size=8, max_slots=4)
    for batch_no, lengths in enumerate([[9, 80, 1, 44], [130, 3, 26], [5, 5, 62, 25]]):
        reqs = prompts_for(_vocab(name), lengths, seed=30 + batch_no)
        decode = [min(k, len(p) - 1) for k, p in zip([6, 40, 0, 9], reqs)]
        heads = [len(p) - k for p, k in zip(reqs, decode)]
        slots = [cache.admit() for _ in reqs]                 # the second and third batch get used slots, states and pages
        got = eng.model.step(cache, slots, [p[:h] for p, h in zip(reqs, heads)], "last")
        for i, (p, h) in enumerate(zip(reqs, heads)):
            assert truth(folders[name], p).excess(got[i], [h - 1], dtype) < 1
        live = [i for i in range(len(reqs)) if heads[i] < len(reqs[i])]
        for i in set(range(len(reqs))) - set(live):
            cache.release(slots[i])
        step = 0
        while live:
            got = eng.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + step]] for i in live], "last")
            for j, i in enumerate(live):
                want = truth(folders[name], reqs[i])
                assert want.excess(got[j], [heads[i] + step], dtype) < 1, f"batch {batch_no}, request {i}, decoded token {step}"
            step += 1
            for i in [i for i in live if heads[i] + step >= len(reqs[i])]:
                cache.release(slots[i])
                live.remove(i)
        cache.check_invariants()
        assert cache.blocks_in_use() == [0] * len(cache.groups)
    eng.model.check_status()


def test_batch_neighbours_change_no_bit_in_float32(engines):
    for name in NAMES:
        eng = engines[(name, "float32")]
        reqs = prompts_for(_vocab(name), [70, 3, 131], seed=40)
        cache = eng.model.new_cache(max_tokens=512, block_size=8, max_slots=4)
        alone = []
        for p in reqs:
            s = cache.admit()
            a = eng.model.step(cache, [s], [p[:-2]], "last").clone()
            b = eng.model.step(cache, [s], [[p[-2]]], "last").clone()
            alone.append((a, b))
            cache.release(s)
        slots = [cache.admit() for _ in reqs]
        a = eng.model.step(cache, slots, [p[:-2] for p in reqs], "last").clone()
        b = eng.model.step(cache, slots, [[p[-2]] for p in reqs], "last").clone()
        for i in range(len(reqs)):
            assert torch.equal(a[i], alone[i][0][0]) and torch.equal(b[i], alone[i][1][0]), f"{name}: request {i}"


@pytest.mark.parametrize("seed", range(100, 124))
def test_configurations_drawn_at_random_in_float32(tmp_path, seed):
    """Sizes and layer orders nobody chose: a whole prompt, then a batch of unequal prompts decoded together, against
    the plain model."""
    cfg = random_config(seed)
    folder = fd.write_random_model(tmp_path / "m", cfg, seed)
    W = weights_of(folder)
    cfg = raw_config(folder)
    reqs = prompts_for(cfg["vocab"], [1, 37, 131], seed=seed)
    want = [Truth(cfg, W, r) for r in reqs]
    eng = fd.load(folder, device="cuda", dtype="float32")
    cache = eng.model.new_cache(max_tokens=256, max_slots=4, slack_blocks=4, block_size=16)
    s = cache.admit()
    assert want[2].excess(eng.model.step(cache, [s], [reqs[2]], "all"), range(len(reqs[2])), "float32") < 1, cfg
    cache.release(s)
    slots = [cache.admit() for _ in reqs]
    heads = [1, 30, 120]
    got = eng.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], "last")
    for i in range(3):
        assert want[i].excess(got[i], [heads[i] - 1], "float32") < 1, cfg
    cache.release(slots[0])
    for step in range(7):
        live = [i for i in (1, 2) if heads[i] + step < len(reqs[i])]
        got = eng.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + step]] for i in live], "last")
        for j, i in enumerate(live):
            assert want[i].excess(got[j], [heads[i] + step], "float32") < 1, (cfg, i, step)
    eng.model.check_status()
    cache.check_invariants()


@pytest.mark.parametrize("seed", range(200, 206))
def test_configurations_drawn_at_random_in_bfloat16(tmp_path, seed):
    cfg = random_config(seed)
    folder = fd.write_random_model(tmp_path / "m", cfg, seed)
    W = weights_of(folder)
    cfg = raw_config(folder)
    reqs = prompts_for(cfg["vocab"], [20, 150], seed=seed)
    want = [Truth(cfg, W, r) for r in reqs]
    eng = fd.load(folder, device="cuda", dtype="bfloat16")
    cache = eng.model.new_cache(max_tokens=256, max_slots=4, slack_blocks=4, block_size=16)
    slots = [cache.admit() for _ in reqs]
    heads = [10, 140]
    got = eng.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], "last")
    for i in range(2):
        assert want[i].excess(got[i], [heads[i] - 1], "bfloat16") < 1, cfg
    for step in range(10):
        got = eng.model.step(cache, slots, [[reqs[i][heads[i] + step]] for i in range(2)], "last")
        for i in range(2):
            assert want[i].excess(got[i], [heads[i] + step], "bfloat16") < 1, (cfg, i, step)
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompts_at_sizes_of_the_tensor_core_kernels(tmp_path, dtype):
    """Heads of 64 on every mixer, prompts of several hundred tokens: many segments of the recurrences, key tiles
    between the kept positions and the window that are never visited, two value heads in one CTA; every position of
    each prompt alone, then the two together and decoded on."""
    import revelix_helpers as H
    rot = H._rot(32, 10000.0, (4.0, 64, 16.0, 1.0))
    att = H.attention(4, 2, 64, 64, 3, 0.125, softcap=15.0, window=150, keep_first=20, rot=rot)
    cfg = H.model(333, 128, 1e-5, [
        H.retention(2, 64, 64, [0.97, 0.999], H._rot(64, 10000.0), H.dense(96)),
        H.parallel(att, H.recurrence(2, 64, 32), 0.7, 1.2, H.dense(96)),
        H.retention(3, 128, 32, [0.9, 0.99, 1.0], H._rot(16, 100.0)),
        H.parallel(att, H.recurrence(1, 128, 64), mlp=H.dense(40))], logit_scale=0.5)
    folder = fd.write_random_model(tmp_path / "m", cfg, 7)
    W = weights_of(folder)
    cfg = raw_config(folder)
    reqs = prompts_for(cfg["vocab"], [610, 333], seed=7)
    want = [Truth(cfg, W, r) for r in reqs]
    eng = fd.load(folder, device="cuda", dtype=dtype)
    cache = eng.model.new_cache(max_tokens=1024, max_slots=4, slack_blocks=4, block_size=64)
    for r, w in zip(reqs, want):
        s = cache.admit()
        assert w.excess(eng.model.step(cache, [s], [r], "all"), range(len(r)), dtype) < 1, f"prompt of {len(r)} tokens"
        cache.release(s)
    slots = [cache.admit() for _ in reqs]
    heads = [600, 325]
    got = eng.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], "last")
    for i in range(2):
        assert want[i].excess(got[i], [heads[i] - 1], dtype) < 1
    for step in range(8):
        got = eng.model.step(cache, slots, [[reqs[i][heads[i] + step]] for i in range(2)], "last")
        for i in range(2):
            assert want[i].excess(got[i], [heads[i] + step], dtype) < 1, (i, step)
    eng.model.check_status()
    cache.check_invariants()


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(folders, name):
    """``Engine.generate``: the scheduler admits five requests three at a time, decode steps replay captured graphs."""
    eng = fd.load(folders[name], device="cuda", dtype="float32")
    prompts = prompts_for(_vocab(name), [3, 30, 1, 70, 9], seed=50)
    got = eng.generate(prompts, 40, max_batch=3)
    for p, r in zip(prompts, got):
        assert r.tokens == plain_greedy(folders[name], p, 40)
    eng.model.check_status()


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_in_bfloat16_picks_a_best_token(folders, name):
    eng = fd.load(folders[name], device="cuda", dtype="bfloat16")
    prompts = prompts_for(_vocab(name), [5, 50, 2], seed=51)
    got = eng.generate(prompts, 30)
    for p, r in zip(prompts, got):
        full = p + r.tokens
        ref = oracle_logits(folders[name], full[:-1])
        scale = float(ref.abs().max())
        for i, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 2 * TOL["bfloat16"] * scale, f"token {i}"
    eng.model.check_status()


def test_command_line_generates(folders):
    p = prompts_for(_vocab("Q"), [12], seed=52)[0]
    cmd = [sys.executable, "-m", "flashdecode_cuda_b200", "generate", "--model", str(folders["Q"]), "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, p)), "--max-new-tokens", "8"]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["tokens"] == plain_greedy(folders["Q"], p, 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_replays_a_schedule(folders, tmp_path, dtype):
    """Prompts of unequal lengths in one step, then one token each, the shorter request ending earlier; the same
    request again afterwards in the freed slot."""
    name = "P"
    a, b = prompts_for(_vocab(name), [40, 9], seed=53)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 23, 24, 29]},
                                     {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[30]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[31]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]}]
    steps += [{"step": 3 + i, "entries": [{"id": "a", "tokens": [a[32 + i]], "want": [0]}], "end": ["a"] if i == 7 else []}
              for i in range(8)]
    steps.append({"step": 11, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]})
    out = tmp_path / "out"
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folders[name]), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", cwd=ROOT,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(12)]
    V = _vocab(name)
    wa, wb = truth(folders[name], a), truth(folders[name], b)

    def read(i):
        return torch.frombuffer(bytearray((out / f"{i}.f32").read_bytes()), dtype=torch.float32).view(-1, V)
    assert wa.excess(read(0)[:4], [0, 23, 24, 29], dtype) < 1 and wb.excess(read(0)[4:], [6], dtype) < 1
    assert wa.excess(read(1), [30], dtype) < 1
    assert wa.excess(read(2)[:1], [31], dtype) < 1 and wb.excess(read(2)[1:], [8], dtype) < 1
    for i in range(8):
        assert wa.excess(read(3 + i), [32 + i], dtype) < 1
    assert wb.excess(read(11), [8], dtype) < 1
