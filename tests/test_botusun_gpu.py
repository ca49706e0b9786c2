"""Botusun on the GPU against the plain implementation: each mechanism's kernels alone, then whole models in float32
and bfloat16 - whole prompts, token-by-token decoding, portions down to two tokens, unequal batches against each
request alone, slots and pages used again, keys far away, at page borders and at the window's edges, long decoding,
greedy generation through the engine's entry point and scheduler, the command line and the trace runner."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200 import kernels as K
from flashdecode_cuda_b200.parts.rope import RotaryScaled
from helpers import prompts_for, rel_err
from botusun_helpers import (BOTUSUN, MODEL_TOL as TOL, Truth, decisive_corrections, oracle_logits, plain_greedy,
                             random_config, raw_config, truth, weights_of, write_folder)
import botusun_helpers as BH
from plain import botusun_plain as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda"
NAMES = ["A", "B", "C"]
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
@pytest.mark.parametrize("scale", [1.0, 12.0, 0.37])
def test_embedding_rows_enter_the_stream_scaled(scale):
    table = torch.randn(50, 72).bfloat16().to(DEV)
    tokens = i32([3, 49, 0, 3])
    resid = torch.zeros(4, 72, device=DEV)
    K.embed(tokens, table, resid, new_status(), scale)
    assert torch.equal(resid.cpu(), table[tokens.long()].float().cpu() * scale)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(1, 64), (5, 100), (37, 1032), (3, 4096 + 8)])
def test_norm_adds_its_delta_times_a_constant(dtype, T, H):
    """resid += c * delta, then the norm: a delta in the model's dtype, a float one, and float partial sums."""
    torch.manual_seed(T + H)
    dt = TD[dtype]
    w = (1 + 0.1 * torch.randn(H)).to(DEV)
    for c in (0.3, 1.0):
        for kind in ("plain", "float", "parts"):
            resid = torch.randn(T, H)
            delta = torch.randn(3, T, H) if kind == "parts" else torch.randn(T, H).to(dt if kind == "plain" else torch.float32)
            total = resid.double() + c * (delta.double().sum(0) if kind == "parts" else delta.double())
            want = P.rms_norm(total, w.double().cpu(), 1e-5)
            r, out = resid.to(DEV), torch.zeros(T, H, dtype=dt, device=DEV)
            K.add_rmsnorm(delta.to(DEV), r, w, 1e-5, out, delta_scale=c)
            assert rel_err(r, total) < 1e-6, (c, kind)
            assert rel_err(out, want) < KTOL[dtype], (c, kind)


@pytest.mark.parametrize("dtype", DTYPES)
def test_pass_vector_is_added_with_the_pending_delta(dtype):
    torch.manual_seed(4)
    T, H = 7, 200
    resid, delta, vec = torch.randn(T, H), torch.randn(T, H).to(TD[dtype]), torch.randn(H)
    r = resid.to(DEV)
    K.add_row_vector(delta.to(DEV), r, vec.to(DEV), 0.3)
    assert rel_err(r, resid.double() + 0.3 * delta.double() + vec.double()) < 1e-6
    r = resid.to(DEV)
    K.add_row_vector(None, r, vec.to(DEV), 0.3)
    assert rel_err(r, resid.double() + vec.double()) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,rot,d,norm,cuts", [(3, 8, 16, True, [5, 1, 1, 6]), (4, 16, 16, True, [2, 2, 9]),
                                                  (1, 0, 32, True, [7, 1]), (2, 32, 32, False, [1, 1, 1, 10]),
                                                  (5, 6, 8, True, [3, 1, 1, 10, 1]), (4, 40, 72, True, [30, 1, 2, 70])])
def test_convolution_head_norm_rotation_and_values_taken_from_the_keys(dtype, taps, rot, d, norm, cuts):
    """Two sequences fed in portions (some of one token, some shorter than the taps): q and the cached keys equal the
    plain convolution, norm per head and rotation of pairs (i, i + rot / 2) with wavelength-scaled frequencies over the
    whole sequences; the cached values equal the convolved keys before norm and rotation; the state is carried."""
    torch.manual_seed(taps * 100 + rot)
    dt = TD[dtype]
    n_q, n_kv, bs, col0 = 4, 2, 4, 10
    C = (n_q + n_kv) * d
    S = sum(cuts)
    lens = [S, S - 3]
    u = [torch.randn(n, col0 + C + 6).to(dt) for n in lens]
    w = torch.randn(C, taps) * 0.5
    qw, kw = (1 + 0.3 * torch.randn(d)), (1 + 0.3 * torch.randn(d))
    n_blocks = -(-S // bs)
    k_pool = torch.zeros(2 * n_blocks + 2, n_kv, bs, d, dtype=dt, device=DEV)
    v_pool = torch.zeros(2 * n_blocks + 2, n_kv, bs, d, dtype=dt, device=DEV)
    table = torch.full((4, n_blocks), -1, dtype=torch.int32, device=DEV)
    slots = [2, 0]
    perm = torch.randperm(2 * n_blocks + 2)
    table[2] = perm[:n_blocks].to(torch.int32).to(DEV)
    table[0] = perm[n_blocks:2 * n_blocks].to(torch.int32).to(DEV)
    state = torch.zeros(4, max(taps - 1, 1), C, device=DEV) if taps > 1 else None
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}
    pos = RotaryScaled(rot, 100.0, sc) if rot else None
    if pos:
        pos.prepare(256, _Rt)
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
                           tok_pos, row_slot, q_start, q_len, k_pool, v_pool, table, n_q, n_kv, d, d, True, single, status,
                           first_col=col0, q_norm=qw.to(DEV) if norm else None, k_norm=kw.to(DEV) if norm else None,
                           norm_eps=1e-5, values_from_keys=True)
        if state is not None and not single:
            K.conv_state_update(proj, state, row_slot, q_start, q_len, len(rows), first_col=col0)
        at = 0
        for r, n in zip(rows, q_lens):
            q_got[r][done[r]:done[r] + n] = q_out[at:at + n].float().cpu()
            at += n
            done[r] += n
    assert int(status.item()) == 0
    fr = P.rot_frequencies(rot, 100.0, sc) if rot else None
    for r in range(2):
        n = lens[r]
        y = P.short_conv(u[r][:, col0:col0 + C].double(), w.double())
        q_want, k_want = y[:, :n_q * d].reshape(n, n_q, d), y[:, n_q * d:].reshape(n, n_kv, d)
        v_want = k_want
        if norm:
            q_want, k_want = P.rms_norm(q_want, qw.double(), 1e-5), P.rms_norm(k_want, kw.double(), 1e-5)
        if rot:
            q_want, k_want = P.rotate_half(q_want, torch.arange(n), rot, fr), P.rotate_half(k_want, torch.arange(n), rot, fr)
        assert rel_err(q_got[r], q_want.reshape(n, -1)) < KTOL[dtype]
        blocks = table[slots[r]].tolist()
        k_got = torch.stack([k_pool[blocks[p // bs], :, p % bs] for p in range(n)]).float().cpu()
        v_got = torch.stack([v_pool[blocks[p // bs], :, p % bs] for p in range(n)]).float().cpu()
        assert rel_err(k_got, k_want) < KTOL[dtype] and rel_err(v_got, v_want) < KTOL[dtype]
        if state is not None:
            assert torch.equal(state[slots[r]].cpu(), u[r][n - (taps - 1):, col0:col0 + C].float())


def test_head_norm_runs_over_the_true_head_size_when_heads_are_padded():
    """A head of 12 dimensions padded to 16 with zero channels: the mean runs over 12."""
    torch.manual_seed(1)
    n_q, n_kv, d, dp, T = 2, 1, 12, 16, 3
    u = torch.zeros(T, (n_q + n_kv) * dp)
    for h in range(n_q + n_kv):
        u[:, h * dp:h * dp + d] = torch.randn(T, d)
    wq = torch.zeros(dp)
    wq[:d] = 1 + 0.2 * torch.randn(d)
    k_pool = torch.zeros(2, n_kv, 4, dp, device=DEV)
    v_pool = torch.zeros(2, n_kv, 4, dp, device=DEV)
    tok_row, tok_pos, row_slot, q_start, q_len, _ = step_arrays([0], [T], [0])
    q_out = torch.zeros(T, n_q * dp, device=DEV)
    K.conv_rope_append(u.to(DEV), torch.ones((n_q + n_kv) * dp, 1, device=DEV), None, q_out, None, None, 0, tok_row, tok_pos,
                       row_slot, q_start, q_len, k_pool, v_pool, i32([[0, 1]]), n_q, n_kv, dp, dp, True, False, new_status(),
                       q_norm=wq.to(DEV), k_norm=wq.to(DEV), norm_eps=1e-6, norm_count=d, values_from_keys=True)
    want = P.rms_norm(u.view(T, n_q + n_kv, dp)[:, :n_q, :d].double(), wq[:d].double(), 1e-6)
    assert rel_err(q_out.view(T, n_q, dp)[:, :, :d], want) < 2e-6
    assert float(q_out.view(T, n_q, dp)[:, :, d:].abs().max()) == 0.0


def _scan_in_portions(dt, proj_of, gate_of, H, d, dv, lens, cuts, tau, segments=False):
    """``K.linear_scan`` with a decay per key channel over two sequences cut into portions; returns (outputs per
    sequence, final states)."""
    slots = [3, 1]
    nk = H * d
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
        gate = torch.cat([gate_of[r][done[r]:done[r] + n] for r, n in zip(rows, q_lens)]).to(DEV).contiguous()
        _, _, row_slot, q_start, q_len, ctx_len = step_arrays([done[r] for r in rows], q_lens, [slots[r] for r in rows])
        out = torch.full((proj.shape[0], H * dv), float("nan"), device=DEV)
        kw = {}
        if segments:
            n_scr = K.linear_scan_scratch_floats(proj.shape[0], len(rows), H, d, dv)
            kw = dict(max_q_len=max(q_lens), scratch=torch.full((n_scr,), float("nan"), device=DEV))
        K.linear_scan(proj, 2, 2 + nk, 2 + 2 * nk, state, out, K.SCAN_CHANNEL_DECAY, row_slot, q_start, q_len, ctx_len,
                      len(rows), H, d, dv, True, status, gate=gate, gate_col=3, q_scale=d ** -0.5, tau=tau, **kw)
        at = 0
        for r, n in zip(rows, q_lens):
            got[r][done[r]:done[r] + n] = out[at:at + n].cpu()
            at += n
            done[r] += n
    assert done == lens and int(status.item()) == 0
    assert bool((state[4] == 7.0).all())
    return got, [state[s].cpu() for s in slots]


SCAN_CASES = [(2, 16, 8, 16.0), (3, 24, 40, 1.0), (1, 64, 64, 4.0), (2, 136, 24, 64.0), (1, 12, 6, 2.0), (4, 128, 128, 16.0),
              (1, 256, 72, 8.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("segments", [False, True])
@pytest.mark.parametrize("H,d,dv,tau", SCAN_CASES)
def test_channel_decay_recurrence_in_portions_and_segments(dtype, H, d, dv, tau, segments):
    """S_t = diag(sigmoid(z_t)^(1/tau)) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_t d^(-1/2)) from portions of many sizes -
    long ones as segments side by side - against the plain token-by-token recurrence over the whole sequences.  The
    pre-activations reach far out on both sides (decays of nearly 0 and of 1 - 1e-9)."""
    if segments and (H, d) not in ((2, 16), (3, 24), (2, 136), (4, 128), (1, 256)):
        pytest.skip("segments are run at a selection of sizes")
    torch.manual_seed(H * d + dv)
    dt = TD[dtype]
    lens, cuts = ([459, 262], [192, 129, 1, 63, 65, 3, 128]) if segments else ([90, 41], [17, 1, 1, 2, 30, 3, 1, 16, 64])
    nk, nv = H * d, H * dv
    proj_of = [torch.randn(n, 2 + 2 * nk + nv + 3).to(dt).float() for n in lens]
    gate_of = [torch.randn(n, 3 + nk + 1) * 6.0 + 3.0 for n in lens]
    got, states = _scan_in_portions(dt, proj_of, gate_of, H, d, dv, lens, cuts, tau, segments)
    for r, n in enumerate(lens):
        x = proj_of[r].double()
        q, k = x[:, 2:2 + nk].reshape(n, H, d) * d ** -0.5, x[:, 2 + nk:2 + 2 * nk].reshape(n, H, d)
        v = x[:, 2 + 2 * nk:2 + 2 * nk + nv].reshape(n, H, dv)
        a = torch.sigmoid(gate_of[r][:, 3:3 + nk].double()).pow(1.0 / tau).reshape(n, H, d)
        want, final = P.channel_decay_recurrence(q, k, v, a)
        assert rel_err(got[r], want.reshape(n, nv)) < 2e-5           # the recurrence is float32 in both dtypes
        assert rel_err(states[r], final) < 2e-5


def _window_case(dtype, d, G, n_kv, window, bs, S, portions, seed, far=False):
    """Keys that stand out: every seventh position (each is the oldest key inside the window of one query and the
    newest outside it for the next) and - with ``far`` - one key hundreds of positions back that only a long window still
    shows.  A window that is one position off, or the keyless term left out of the denominator, changes the result by
    the size of a value."""
    torch.manual_seed(seed)
    dt = TD[dtype]
    n_q = G * n_kv
    q = torch.randn(S, n_q, d) * 0.3
    k = torch.randn(S, n_kv, d) * 0.3
    v = torch.randn(S, n_kv, d)
    e = torch.zeros(d)
    e[3 % d] = 1.0
    for p in {p for p in range(S) if p % 7 == 0} | ({2} if far else set()):
        k[p] += 6.0 * e
    q += 2.0 * e
    q[S // 2:] *= 0.05                 # the second half's scores are small: the keyless term is most of the denominator
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    scale = 0.7
    want = P.sink_softmax_attention(q.double(), k.double(), v.double(), scale, window).reshape(S, n_q * d)
    n_cols = -(-S // bs)
    k_pool = torch.zeros(n_cols + 3, n_kv, bs, d, dtype=dt, device=DEV)
    v_pool = torch.zeros(n_cols + 3, n_kv, bs, d, dtype=dt, device=DEV)
    perm = torch.randperm(n_cols + 3)[:n_cols]
    table = torch.full((2, n_cols), -1, dtype=torch.int32, device=DEV)
    table[1] = perm.to(torch.int32).to(DEV)
    for p in range(S):
        k_pool[perm[p // bs], :, p % bs] = k[p].to(DEV)
        v_pool[perm[p // bs], :, p % bs] = v[p].to(DEV)
    status = new_status()
    sink = torch.zeros(n_q, device=DEV)
    got = torch.zeros(S, n_q * d)
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
            scratch = torch.zeros(K.attention_scratch_floats(1, n_q, d, n_splits), device=DEV)
        out = torch.full((n, n_q * d), float("nan"), dtype=dt, device=DEV)
        K.attention_ext(q[at:at + n].reshape(n, n_q * d).to(DEV).contiguous(), k_pool, v_pool, out, table, tok_row, row_slot,
                        q_start, q_len, ctx_len, 1, n, n_q, n_kv, d, scale, window or 0, n_splits, split_len, scratch, status,
                        sink=sink)
        got[at:at + n] = out.float().cpu()
        at += n
    assert at == S and int(status.item()) == 0
    err = (got.double() - want).abs().max(dim=1).values / want.abs().max()
    assert float(err.max()) < KTOL[dtype], f"first wrong position {int((err >= KTOL[dtype]).nonzero()[0])} (window {window})"


WINDOW_CASES = [  # d, G, n_kv, window, block size, length
    (16, 2, 2, 7, 4, 60), (64, 4, 2, 21, 16, 150), (24, 3, 1, 1, 8, 40), (128, 2, 1, 64, 64, 200), (40, 1, 3, 14, 7, 90),
    (64, 8, 1, None, 16, 100), (32, 2, 2, 500, 8, 330)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", WINDOW_CASES)
def test_windowed_attention_with_the_unit_sink_whole_prompt(dtype, case):
    d, G, n_kv, window, bs, S = case
    _window_case(dtype, d, G, n_kv, window, bs, S, [S], seed=11, far=window is None or window > 300)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", WINDOW_CASES)
def test_windowed_attention_with_the_unit_sink_in_portions_and_token_by_token(dtype, case):
    d, G, n_kv, window, bs, S = case
    _window_case(dtype, d, G, n_kv, window, bs, S, [5, 2, 1, 1, 17, 3] + [1] * 400, seed=12, far=window is None or window > 300)


ROUTE_CASES = [  # router outputs, top, groups (count, keep), weight scale, correction spread
    (8, 2, (4, 3), 2.0, 0.02), (6, 3, (2, 1), 0.5, 0.5), (4, 1, (4, 2), 1.0, 0.3), (12, 4, (3, 3), 1.0, 0.1),
    (5, 2, None, 2.5, 0.2), (64, 8, (8, 4), 1.0, 0.05), (9, 3, (3, 1), 1.0, 0.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ROUTE_CASES)
@pytest.mark.parametrize("T", [3, 70])
def test_sigmoid_scores_and_the_choice_among_the_best_groups(dtype, case, T):
    """ids and weights against the plain routing, with the logits made by the kernel itself and given to it.  A second
    run shifts every correction far below zero: choice scores are negative, and experts outside the kept groups must
    still lose (they count as minus infinity, not as zero)."""
    E, top, groups, ws, spread = case
    torch.manual_seed(E * 10 + top)
    dt = TD[dtype]
    H = 96
    x = torch.randn(T, H).to(dt)
    router = (torch.randn(E, H) / H ** 0.5 * 3).to(dt)
    rc = {"experts": E, "top": top, "scale": ws}
    if groups:
        rc["groups"] = {"count": groups[0], "keep": groups[1]}
    for shift in (0.0, -5.0):
        corr = torch.randn(E) * spread + shift
        want_ids, want_w = P.route(x.double(), router.double(), corr.double(), rc)
        for given in (False, True):
            ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
            wts = torch.zeros(T, top, device=DEV)
            logits = (x.float() @ router.float().T).to(DEV) if given else None
            K.moe_route(x.to(DEV), router.to(DEV), corr.to(DEV), ids, wts, logits, sigmoid_scores=True,
                        n_groups=groups[0] if groups else 1, keep_groups=groups[1] if groups else 1, weight_scale=ws)
            order = ids.long().cpu().sort(dim=1)
            want_order = want_ids.sort(dim=1)
            # a token whose two best candidates lie closer than rounding may fall either way: none among these
            assert torch.equal(order.values, want_order.values), (case, shift, given)
            assert rel_err(wts.cpu().gather(1, order.indices), want_w.gather(1, want_order.indices)) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,dim", [(1, 64, 16), (5, 100, 4), (64, 256, 20), (65, 256, 20), (300, 1032, 32), (7, 72, 1)])
def test_token_side_input_for_few_tokens_and_as_separate_kernels(dtype, T, H, dim):
    """out = unit_rms(P (gelu(G x) * e)) * w with x = resid + c * delta completed on the way, against the plain
    function: the form for steps of few tokens (bfloat16) and the form whose products are matrix products."""
    torch.manual_seed(T + H + dim)
    dt = TD[dtype]
    V, layers, layer, c = 37, 3, 1, 0.3
    table = torch.randn(V, layers * dim).to(dt)
    G, Pm = (torch.randn(dim, H) / H ** 0.5).to(dt), (torch.randn(H, dim) / dim ** 0.5).to(dt)
    w = 1 + 0.1 * torch.randn(H)
    tokens = torch.randint(0, V, (T,))
    resid, delta = torch.randn(T, H) * 3, torch.randn(T, H).to(dt)
    x = resid.double() + c * delta.double()
    Wd = {"side.embed": table.double(), "l1.side.gate": G.double(), "l1.side.proj": Pm.double(), "l1.side.norm": w.double()}
    x_in = x.to(dt).double() if dtype == "bfloat16" else x          # the product's operand is the stream in the model's dtype
    want = P.token_side(x_in, tokens, Wd, layer, dim, 1e-5)
    status = new_status()
    forms = ["separate"] + (["few launches"] if T <= 64 and dtype == "bfloat16" else [])
    from flashdecode_cuda_b200.parts.linear import matmul
    for form in forms:
        r, out = resid.to(DEV), torch.full((T, H), float("nan"), device=DEV)
        if form == "few launches":
            K.token_side_row(delta.to(DEV), r, c, i32(tokens.tolist()), table.to(DEV), layer * dim, G.to(DEV), Pm.to(DEV),
                             w.to(DEV), 1e-5, out, status)
        else:
            xs = torch.zeros(T, H, dtype=dt, device=DEV)
            K.add_cast(delta.to(DEV), r, xs, c)
            z = torch.zeros(T, dim, device=DEV)
            matmul(xs, G.to(DEV), None, z)
            g = torch.zeros(T, dim, dtype=dt, device=DEV)
            K.side_gate_mul(z, i32(tokens.tolist()), table.to(DEV), layer * dim, g, status)
            y = torch.zeros(T, H, device=DEV)
            matmul(g, Pm.to(DEV), None, y)
            K.add_rmsnorm(None, y, w.to(DEV), 1e-5, out, write_resid=False)
        assert rel_err(r, x) < 1e-6, form
        assert rel_err(out, want) < (3e-2 if dtype == "bfloat16" else 2e-5), form
    assert int(status.item()) == 0


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("botusun")
    out = {(n, "float32"): write_folder(tmp, n, seed=31) for n in NAMES}
    # bfloat16: the corrections alone decide the routers' choices
    out.update({(n, "bfloat16"): write_folder(tmp, n, seed=31, decisive=True) for n in NAMES})
    return out


@pytest.fixture(scope="module")
def engines(folders):
    return {(n, d): fd.load(folders[(n, d)], device="cuda", dtype=d) for n in NAMES for d in DTYPES}


def _vocab(name):
    return BOTUSUN[name]["vocab"]


def _lengths(name):
    # around the windows (27, 40 / 16 / 1), the taps and the pages
    return {"A": [1, 2, 3, 27, 28, 40, 41, 75, 140], "B": [1, 16, 17, 64, 65, 129], "C": [1, 2, 5, 6, 24, 100, 201]}[name]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("block_size", [8, 64])
def test_whole_prompts(engines, folders, name, dtype, block_size):
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=320, block_size=block_size)
    for p in prompts_for(_vocab(name), _lengths(name), seed=1):
        slot = cache.admit()
        got = eng.model.step(cache, [slot], [p], "all")
        assert truth(folders[(name, dtype)], p).excess(got, range(len(p)), dtype) < 1, f"prompt of {len(p)} tokens"
        cache.release(slot)
    eng.model.check_status()
    cache.check_invariants()


def test_every_layer_run_in_float32(engines, folders):
    """The residual stream after every layer run (a looped layer counts each time) against the plain one."""
    for name in NAMES:
        eng = engines[(name, "float32")]
        folder = folders[(name, "float32")]
        (p,) = prompts_for(_vocab(name), [45], seed=2)
        _, layers = P.forward(raw_config(folder), weights_of(folder), p, return_layers=True)
        cache = eng.model.new_cache(max_tokens=64)
        slot = cache.admit()
        eng.model.trace = {}
        eng.model.step(cache, [slot], [p], None)
        got, eng.model.trace = eng.model.trace, None
        assert len(layers) == len(eng.model.schedule)
        for i, want in enumerate(layers):
            assert rel_err(got[f"layer.{i}"], want) < 1e-5, f"{name}: layer run {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_token_by_token_across_window_edges(engines, folders, name, dtype):
    """A prompt of one token or of thirty, then so many single tokens that every window of the model passes over
    decoded tokens."""
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=256, block_size=16)
    n_decode = {"A": 70, "B": 45, "C": 40}[name]
    for head in (1, 30):
        (p,) = prompts_for(_vocab(name), [head + n_decode], seed=3 + head)
        want = truth(folders[(name, dtype)], p)
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
    windows' pages are given back and used again."""
    name = "A"
    eng = engines[(name, "float32")]
    (p,) = prompts_for(_vocab(name), [420], seed=9)
    want = oracle_logits(folders[(name, "float32")], p)
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
    want = truth(folders[(name, dtype)], p)
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
    folder = folders[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=64 * 8, block_size=8, max_slots=4)
    for batch_no, lengths in enumerate([[9, 80, 1, 44], [130, 3, 26], [5, 5, 62, 25]]):
        reqs = prompts_for(_vocab(name), lengths, seed=30 + batch_no)
        decode = [min(k, len(p) - 1) for k, p in zip([6, 40, 0, 9], reqs)]
        heads = [len(p) - k for p, k in zip(reqs, decode)]
        slots = [cache.admit() for _ in reqs]                 # the second and third batch get used slots, states and pages
        got = eng.model.step(cache, slots, [p[:h] for p, h in zip(reqs, heads)], "last")
        for i, (p, h) in enumerate(zip(reqs, heads)):
            assert truth(folder, p).excess(got[i], [h - 1], dtype) < 1
        live = [i for i in range(len(reqs)) if heads[i] < len(reqs[i])]
        for i in set(range(len(reqs))) - set(live):
            cache.release(slots[i])
        step = 0
        while live:
            got = eng.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + step]] for i in live], "last")
            for j, i in enumerate(live):
                want = truth(folder, reqs[i])
                assert want.excess(got[j], [heads[i] + step], dtype) < 1, f"batch {batch_no}, request {i}, decoded token {step}"
            step += 1
            for i in [i for i in live if heads[i] + step >= len(reqs[i])]:
                cache.release(slots[i])
                live.remove(i)
        cache.check_invariants()
        assert cache.blocks_in_use() == [0] * len(cache.groups)
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_dozen_requests_decoded_together(engines, folders, dtype):
    """More rows than the register-fed products take: the step's products, the routing and the side input run in their
    forms for 17 to 128 rows; every request's logits equal those of the request alone."""
    name = "A"
    eng, folder = engines[(name, dtype)], folders[(name, dtype)]
    reqs = prompts_for(_vocab(name), [3 + (7 * i) % 45 for i in range(24)], seed=60)
    heads = [max(1, len(p) - 4) for p in reqs]
    cache = eng.model.new_cache(max_tokens=64 * 24, block_size=16, max_slots=24)
    slots = [cache.admit() for _ in reqs]
    got = eng.model.step(cache, slots, [p[:h] for p, h in zip(reqs, heads)], "last")
    for i, (p, h) in enumerate(zip(reqs, heads)):
        assert truth(folder, p).excess(got[i], [h - 1], dtype) < 1, f"request {i}"
    for step in range(3):
        live = [i for i in range(24) if heads[i] + step < len(reqs[i])]
        got = eng.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + step]] for i in live], "last")
        for j, i in enumerate(live):
            assert truth(folder, reqs[i]).excess(got[j], [heads[i] + step], dtype) < 1, f"request {i}, decoded token {step}"
    eng.model.check_status()
    cache.check_invariants()


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


@pytest.mark.parametrize("seed", range(100, 130))
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


@pytest.mark.parametrize("seed", range(200, 208))
def test_configurations_drawn_at_random_in_bfloat16(tmp_path, seed):
    cfg = random_config(seed)
    folder = decisive_corrections(fd.write_random_model(tmp_path / "m", cfg, seed))
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
    """Heads of 64 and 128, a width and experts wide enough for the grouped tcgen05 products with the gate in their
    epilogue, prompts of several hundred tokens:
    many segments of the recurrence, windows that leave most key tiles unvisited, a key far back under a long window;
    every position of each prompt alone, then the two together and decoded on."""
    cfg = BH.model(333, 256, 1e-5, [
        BH.gla(2, 64, 64, 16.0, 16, BH.dense(96)),
        BH.attention(4, 2, 64, 3, 0.125, window=150, rotation=BH.rot(32, 10000.0, (4.0, 1.0, 4.0, 64)),
                     mlp=BH.moe(8, 2, 128, groups=(4, 2), scale=1.5)),
        BH.gla(3, 128, 32, 4.0, 8),
        BH.attention(2, 1, 128, 4, 0.09, window=500, rotation=BH.rot(128, 500000.0), mlp=BH.dense(40))],
        mult=0.5, emb_scale=4.0, side=16, loop=(1, 3, 2))
    folder = fd.write_random_model(tmp_path / "m", cfg, 7)
    if dtype == "bfloat16":
        decisive_corrections(folder)
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
    folder = folders[(name, "float32")]
    eng = fd.load(folder, device="cuda", dtype="float32")
    prompts = prompts_for(_vocab(name), [3, 30, 1, 70, 9], seed=50)
    got = eng.generate(prompts, 40, max_batch=3)
    for p, r in zip(prompts, got):
        assert r.tokens == plain_greedy(folder, p, 40)
    eng.model.check_status()


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_in_bfloat16_picks_a_best_token(folders, name):
    folder = folders[(name, "bfloat16")]
    eng = fd.load(folder, device="cuda", dtype="bfloat16")
    prompts = prompts_for(_vocab(name), [5, 50, 2], seed=51)
    got = eng.generate(prompts, 30)
    for p, r in zip(prompts, got):
        full = p + r.tokens
        ref = oracle_logits(folder, full[:-1])
        scale = float(ref.abs().max())
        for i, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 2 * TOL["bfloat16"] * scale, f"token {i}"
    eng.model.check_status()


def test_command_line_generates(folders):
    folder = folders[("B", "float32")]
    p = prompts_for(_vocab("B"), [12], seed=52)[0]
    cmd = [sys.executable, "-m", "flashdecode_cuda_b200", "generate", "--model", str(folder), "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, p)), "--max-new-tokens", "8"]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["tokens"] == plain_greedy(folder, p, 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_replays_a_schedule(folders, tmp_path, dtype):
    """Prompts of unequal lengths in one step, then one token each, the shorter request ending earlier; the same
    request again afterwards in the freed slot."""
    name = "A"
    folder = folders[(name, dtype)]
    a, b = prompts_for(_vocab(name), [40, 9], seed=53)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 23, 24, 29]},
                                     {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[30]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[31]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]}]
    steps += [{"step": 3 + i, "entries": [{"id": "a", "tokens": [a[32 + i]], "want": [0]}], "end": ["a"] if i == 7 else []}
              for i in range(8)]
    steps.append({"step": 11, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]})
    out = tmp_path / "out"
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", cwd=ROOT,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(12)]
    V = _vocab(name)
    wa, wb = truth(folder, a), truth(folder, b)

    def read(i):
        return torch.frombuffer(bytearray((out / f"{i}.f32").read_bytes()), dtype=torch.float32).view(-1, V)
    assert wa.excess(read(0)[:4], [0, 23, 24, 29], dtype) < 1 and wb.excess(read(0)[4:], [6], dtype) < 1
    assert wa.excess(read(1), [30], dtype) < 1
    assert wa.excess(read(2)[:1], [31], dtype) < 1 and wb.excess(read(2)[1:], [8], dtype) < 1
    for i in range(8):
        assert wa.excess(read(3 + i), [32 + i], dtype) < 1
    assert wb.excess(read(11), [8], dtype) < 1
