"""Ropulix through the framework against the plain implementation: every mechanism's kernels alone (with inputs made so
that a key at a window's edge, a far key or a page border shows), then whole models under every way of cutting the work
(whole prompts, decoding token by token, portions down to two tokens, mixed batches whose pages and slots are used
again), in 32-bit and in bfloat16, and greedy generation through the engine's own entry point."""

import math
import random

import numpy as np
import pytest
import torch

from tests import helpers
from tests.plain import ropulix_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
# a row of logits against the plain model in 64-bit, as fractions of the row's root mean square: (rms, largest).
# float32 is the sharp comparison.  bfloat16: the plain model rounds its activations where the engine stores them; a
# rounding that falls the other way moves single rows by several per cent, so a request passes when at most a tenth of its
# rows (or one) is beyond BF16_USUAL and none beyond BF16_WORST.  A row at which some router's last chosen logit lies within
# CLOSE_CALL of the first one left out is not compared: there the two models may rightly send the token to different experts.
# A wrong state, slot or page moves every row after it; the kernels alone are compared sharply above.
TOL = {"float32": (3e-5, 2e-4)}
BF16_USUAL, BF16_WORST, CLOSE_CALL = 6e-2, 5e-1, 0.15


def dev(t):
    return t.to(DEV)


def _pages(seed, page, lengths, spare=3):
    """Block tables that scatter each sequence over pages in a shuffled order; returns (table, pages in use)."""

    rng = random.Random(seed)
    need = [-(-n // page) for n in lengths]
    ids = list(range(sum(need) + spare))
    rng.shuffle(ids)
    table = torch.full((len(lengths), max(need)), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(need):
        table[r, :n] = torch.tensor(ids[at:at + n], dtype=torch.int32)
        at += n
    return table, len(ids)


def _batch(lengths):
    positions = torch.cat([torch.arange(m) for m in lengths]).int()
    entry = torch.cat([torch.full((m,), i) for i, m in enumerate(lengths)]).int()
    return positions, entry


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,dv,page,normalise", [(4, 2, 16, 24, 4, True), (3, 3, 12, 12, 16, True), (2, 1, 40, 8, 8, False)])
def test_head_norm_write_and_windowed_attention(dtype, nq, nkv, d, dv, page, normalise):
    """Unit-norm q and k per head, the page write, and attention under a window, for two sequences in one batch."""

    from llm_runtime_study_b200.ops import functional as F
    from llm_runtime_study_b200.ops import mixer_steps as M

    torch.manual_seed(d + dv)
    lengths, window, eps, scale = [41, 7], 6, 1e-5, 0.6
    n = sum(lengths)
    rows = torch.randn(n, nq * d + nkv * (d + dv) + 5).to(dtype)
    table, pages = _pages(n, page, lengths)
    positions, entry = _batch(lengths)
    k_pool = torch.zeros(pages, nkv, page, d, dtype=dtype, device=DEV)
    v_pool = torch.zeros(pages, nkv, page, dv, dtype=dtype, device=DEV)
    q = M.head_norm_write(dev(rows), num_q_heads=nq, num_kv_heads=nkv, head_dim=d, value_dim=dv, eps=eps, normalise=normalise,
                          positions=dev(positions), token_entry=dev(entry), block_table=dev(table), page_size=page,
                          k_pool=k_pool, v_pool=v_pool)
    out = F.paged_attention_simt_rules(q, k_pool, v_pool, positions=dev(positions), token_entry=dev(entry), block_table=dev(table),
                                       scale=scale, window=window).cpu().double()
    at = 0
    for m in lengths:
        x = rows[at:at + m].double()
        pq, pk = x[:, : nq * d].view(m, nq, d), x[:, nq * d : (nq + nkv) * d].view(m, nkv, d)
        if normalise:
            pq, pk = plain.unit(pq, eps), plain.unit(pk, eps)
        pv = x[:, (nq + nkv) * d : (nq + nkv) * d + nkv * dv].view(m, nkv, dv)
        if dtype == torch.bfloat16:
            pq, pk = pq.bfloat16().double(), pk.bfloat16().double()
        assert (q[at:at + m].cpu().double() - pq).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2)
        want = plain.softmax_attention(pq, pk, pv, scale=scale, window=window)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert (out[at:at + m] - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
        at += m


def _latent_case(dtype, heads, rank, rot, page, length, window, marked=None, seed=0):
    """Rows ``[c | k_rot]`` for one sequence in scattered pages and queries for its last ``new`` positions; ``marked``
    makes one key stand out: every query points at it, so whether it is seen decides the output."""

    torch.manual_seed(seed)
    d = rank + rot
    rows = 0.3 * torch.randn(length, d)
    q = 0.3 * torch.randn(length, heads, d)
    if marked is not None:
        rows[marked] = 0.0
        rows[marked, 1] = 4.0
        q[:, :, 1] = 4.0
    rows, q = rows.to(dtype), q.to(dtype)
    table, pages = _pages(seed + length, page, [length])
    pool = torch.zeros(pages, page, d, dtype=dtype)
    for t in range(length):
        pool[table[0, t // page], t % page] = rows[t]
    return q, rows, pool, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rank,rot,page,window", [(3, 40, 8, 4, 9), (2, 24, 16, 16, 0), (5, 72, 0, 8, 33), (1, 300, 20, 16, 64)])
def test_latent_attention_over_shared_rows(dtype, heads, rank, rot, page, window):
    """Every head attends over one row per token whose leading columns are also the values."""

    from llm_runtime_study_b200.ops import functional as F

    length = 150
    q, rows, pool, table = _latent_case(dtype, heads, rank, rot, page, length, window, seed=rank)
    positions, entry = _batch([length])
    out = F.paged_attention_simt_latent(dev(q), dev(pool), value_dim=rank, positions=dev(positions), token_entry=dev(entry),
                                        block_table=dev(table), scale=0.2, window=window).cpu().double()
    k = rows.double()[:, None, :]
    want = plain.softmax_attention(q.double(), k, k[:, :, :rank], scale=0.2, window=window or None)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (out - want).abs().max() <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("page,window,marked", [(16, 40, 15), (16, 40, 16), (8, 9, 63), (4, 5, 100), (16, 0, 3)])
def test_a_key_at_the_windows_edge_and_a_far_key(dtype, page, window, marked):
    """One key stands out.  Queries up to ``window - 1`` positions behind it give nearly its value, the next one does not;
    without a window a key hundreds of positions back is found.  The marked key sits at a page's border in several cases."""

    from llm_runtime_study_b200.ops import functional as F

    heads, rank, rot, length = 2, 16, 8, 700
    q, rows, pool, table = _latent_case(dtype, heads, rank, rot, page, length, window, marked=marked, seed=marked)
    positions, entry = _batch([length])
    out = F.paged_attention_simt_latent(dev(q), dev(pool), value_dim=rank, positions=dev(positions), token_entry=dev(entry),
                                        block_table=dev(table), scale=1.0, window=window).cpu().double()
    value = rows[marked, :rank].double()
    last_seen = marked + window - 1 if window else length - 1
    for p in (marked, last_seen - 1, last_seen):
        assert (out[p] - value).abs().max() < 0.05, (p, out[p, 0, :3])
    if window:
        for p in (last_seen + 1, last_seen + 2):
            assert (out[p, :, 1] - 4.0).abs().min() > 2.0, p
    k = rows.double()[:, None, :]
    want = plain.softmax_attention(q.double(), k, k[:, :, :rank], scale=1.0, window=window or None)
    assert (out - want).abs().max() <= (2e-5 if dtype == torch.float32 else 3e-2)


def _latent_ctx(lengths, q_lens):
    """What the kernel chooser reads of a step's context: every sequence of ``lengths`` brings its last ``q_lens`` tokens."""

    from types import SimpleNamespace

    positions = torch.cat([torch.arange(m - k, m) for m, k in zip(lengths, q_lens)]).int()
    entry = torch.cat([torch.full((k,), i) for i, k in enumerate(q_lens)]).int()
    return SimpleNamespace(positions=dev(positions), token_entry=dev(entry), all_decode=max(q_lens) == 1, num_entries=len(lengths),
                           q_lens=list(q_lens), kv_lens=list(lengths), max_kv_len=max(lengths)), positions, entry


@pytest.mark.parametrize("heads,rank,rot,page,window", [(3, 32, 16, 4, 9), (6, 64, 16, 16, 40), (16, 128, 64, 16, 0), (70, 48, 0, 8, 33),
                                                        (5, 512, 64, 16, 100)])
@pytest.mark.parametrize("q_lens", [[150, 41], [1, 1], [2, 37]])
def test_tensor_core_latent_attention(heads, rank, rot, page, window, q_lens):
    """The mma.sync kernel for prompt portions behind cached tokens and for single tokens, several tokens and head groups a
    tile, against the plain attention of each sequence."""

    from llm_runtime_study_b200.ops import attention_latent

    torch.manual_seed(rank + heads)
    lengths, d = [150, 41], rank + rot
    assert attention_latent.supported(rank, rot)
    table, pages = _pages(rank, page, lengths)
    rows = [0.5 * torch.randn(m, d).bfloat16() for m in lengths]
    pool = torch.zeros(pages, page, d, dtype=torch.bfloat16)
    for e, m in enumerate(lengths):
        for t in range(m):
            pool[table[e, t // page], t % page] = rows[e][t]
    ctx, positions, entry = _latent_ctx(lengths, q_lens)
    q = (0.5 * torch.randn(sum(q_lens), heads, d)).bfloat16()
    got = attention_latent.latent_attention(dev(q), dev(pool), ctx, dev(table), value_dim=rank, scale=0.3, window=window).cpu().double()
    at = 0
    for e, (m, k) in enumerate(zip(lengths, q_lens)):
        full_q = torch.zeros(m, heads, d, dtype=torch.float64)
        full_q[m - k:] = q[at:at + k].double()
        keys = rows[e].double()[:, None, :]
        want = plain.softmax_attention(full_q, keys, keys[:, :, :rank], scale=0.3, window=window or None)[m - k:]
        assert (got[at:at + k] - want).abs().max() <= 2e-2 * max(1.0, float(want.abs().max())), (e, float((got[at:at + k] - want).abs().max()))
        at += k


def test_single_tokens_whose_keys_are_cut_into_parts():
    """Three requests of unequal length, one token each: the longest is cut into several parts and merged; a part may
    hold no visible key at all (the short request)."""

    from llm_runtime_study_b200.ops import attention_latent

    torch.manual_seed(8)
    heads, rank, rot, page = 6, 64, 16, 16
    lengths, d = [1500, 3, 700], rank + rot
    for window in (0, 600):
        assert attention_latent.decode_splits(len(lengths), heads, min(window, max(lengths)) if window else max(lengths)) > 1
        table, pages = _pages(window, page, lengths)
        rows = [0.5 * torch.randn(m, d).bfloat16() for m in lengths]
        pool = torch.zeros(pages, page, d, dtype=torch.bfloat16)
        for e, m in enumerate(lengths):
            for t in range(m):
                pool[table[e, t // page], t % page] = rows[e][t]
        ctx, _, _ = _latent_ctx(lengths, [1, 1, 1])
        q = (0.5 * torch.randn(3, heads, d)).bfloat16()
        got = attention_latent.latent_attention(dev(q), dev(pool), ctx, dev(table), value_dim=rank, scale=0.3, window=window).cpu().double()
        for e, m in enumerate(lengths):
            full_q = torch.zeros(m, heads, d, dtype=torch.float64)
            full_q[m - 1] = q[e].double()
            keys = rows[e].double()[:, None, :]
            want = plain.softmax_attention(full_q, keys, keys[:, :, :rank], scale=0.3, window=window or None)[m - 1]
            assert (got[e] - want).abs().max() <= 2e-2 * max(1.0, float(want.abs().max())), (window, e)


@pytest.mark.parametrize("page,window,marked", [(16, 40, 15), (16, 40, 16), (8, 9, 63), (4, 5, 100), (16, 0, 3), (16, 64, 31), (16, 33, 32)])
@pytest.mark.parametrize("new", [700, 1])
def test_tensor_core_latent_attention_at_the_windows_edge(page, window, marked, new):
    """One key stands out, in a whole prompt and for single tokens fed behind cached ones: the last position that sees it gives
    nearly its value, the next one does not; without a window a key hundreds of positions back is found."""

    from llm_runtime_study_b200.ops import attention_latent

    heads, rank, rot, length = 2, 16, 16, 700
    q, rows, pool, table = _latent_case(torch.bfloat16, heads, rank, rot, page, length, window, marked=marked, seed=marked)
    last_seen = marked + window - 1 if window else length - 1
    k = rows.double()[:, None, :]
    want = plain.softmax_attention(q.double(), k, k[:, :, :rank], scale=1.0, window=window or None)
    value = rows[marked, :rank].double()
    if new == length:
        ctx, _, _ = _latent_ctx([length], [length])
        out = attention_latent.latent_attention(dev(q), dev(pool), ctx, dev(table), value_dim=rank, scale=1.0, window=window).cpu().double()
        probes = {p: out[p] for p in (marked, last_seen - 1, last_seen, min(last_seen + 1, length - 1), min(last_seen + 2, length - 1))}
        assert (out - want).abs().max() <= 3e-2
    else:
        probes = {}
        for p in (marked, last_seen - 1, last_seen, min(last_seen + 1, length - 1), min(last_seen + 2, length - 1)):
            ctx, _, _ = _latent_ctx([p + 1], [1])
            probes[p] = attention_latent.latent_attention(dev(q[p:p + 1].contiguous()), dev(pool), ctx, dev(table), value_dim=rank, scale=1.0,
                                                          window=window).cpu().double()[0]
            assert (probes[p] - want[p]).abs().max() <= 3e-2
    for p, row in probes.items():
        if p <= last_seen:
            assert (row - value).abs().max() < 0.05, p
        else:
            assert (row[:, 1] - 4.0).abs().min() > 2.0, p


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_rank,kv_rank,rot,rot_dims,page", [(48, 40, 8, 8, 4), (12, 24, 16, 16, 16), (20, 8, 12, 8, 8)])
def test_latent_rows_and_rotations(dtype, q_rank, kv_rank, rot, rot_dims, page):
    """The normed query latent, the normed latent and rotated key part in the pages, and the rotation of a slice of every head."""

    from llm_runtime_study_b200.ops import mixer_steps as M

    torch.manual_seed(q_rank)
    lengths = [19, 6]
    n = sum(lengths)
    eps, base = 1e-5, 1000.0
    rows = torch.randn(n, q_rank + kv_rank + rot + 3).to(dtype)
    qw, kw = 1 + 0.1 * torch.randn(q_rank), 1 + 0.1 * torch.randn(kv_rank)
    inv_freq = (1.0 / (base ** (torch.arange(0, rot_dims, 2, dtype=torch.float32) / rot_dims)))
    table, pages = _pages(n, page, lengths)
    positions, entry = _batch(lengths)
    # the batch's positions start behind 100 and 3 cached tokens
    starts = [100, 3]
    positions = positions + torch.tensor(starts, dtype=torch.int32)[entry.long()]
    table, pages = _pages(n, page, [s + m for s, m in zip(starts, lengths)])
    pool = torch.zeros(pages, page, kv_rank + rot, dtype=dtype, device=DEV)
    cq = M.latent_prepare(dev(rows), q_offset=0, q_rank=q_rank, q_weight=dev(qw), eps=eps, positions=dev(positions),
                          token_entry=dev(entry), kv_offset=q_rank, kv_rank=kv_rank, kv_weight=dev(kw), rot=rot, rot_dims=rot_dims,
                          inv_freq=dev(inv_freq), block_table=dev(table), page_size=page, pool=pool).cpu().double()
    x = rows.double()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (cq - plain.rms_norm(x[:, :q_rank], qw.double(), eps)).abs().max() <= tol * 4
    want_c = plain.rms_norm(x[:, q_rank : q_rank + kv_rank], kw.double(), eps)
    want_r = plain.rotate_half(x[:, q_rank + kv_rank : q_rank + kv_rank + rot], positions, base, rot_dims)
    for t in range(n):
        p = int(positions[t])
        got = pool[table[int(entry[t]), p // page], p % page].cpu().double()
        assert (got[:kv_rank] - want_c[t]).abs().max() <= tol * 4, t
        assert (got[kv_rank:] - want_r[t]).abs().max() <= tol * 4, t
    heads, head, off = 3, 10 + rot, 10
    src = torch.randn(n, heads * head).to(dtype)
    dst = torch.zeros(n, heads * (5 + rot), dtype=dtype, device=DEV)
    M.rope_slice(dev(src), dst, heads=heads, src_head=head, src_offset=off, dst_head=5 + rot, dst_offset=5, rot=rot, rot_dims=rot_dims,
                 inv_freq=dev(inv_freq), positions=dev(positions))
    want = plain.rotate_half(src.double().view(n, heads, head)[..., off:], positions, base, rot_dims)
    got = dst.cpu().double().view(n, heads, 5 + rot)
    assert (got[..., 5:] - want).abs().max() <= tol * 4 and got[..., :5].abs().max() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gates_and_the_norm_on_a_sublayers_output(dtype):
    from llm_runtime_study_b200.ops import mixer_steps as M

    torch.manual_seed(1)
    x, gate_rows = torch.randn(6, 4 * 24).to(dtype), torch.randn(6, 110).to(dtype)
    got = M.sigmoid_gate(dev(x), dev(gate_rows), gate_offset=7, group=24).cpu().double()
    want = (x.double().view(6, 4, 24) * plain.sigmoid(gate_rows.double()[:, 7:11])[:, :, None]).reshape(6, -1)
    tol = 1e-6 if dtype == torch.float32 else 2e-2
    assert (got - want).abs().max() <= tol
    got = M.sigmoid_gate(dev(x), dev(gate_rows), gate_offset=3, group=1).cpu().double()
    assert (got - x.double() * plain.sigmoid(gate_rows.double()[:, 3:99])).abs().max() <= tol
    out, w, resid = 3 * torch.randn(5, 56), torch.randn(56), torch.randn(5, 56)
    on_dev = dev(resid.clone())
    rounded = M.norm_accumulate_round(dev(out), dev(w), 1e-5, on_dev, dtype if dtype != torch.float32 else None)
    want = resid.double() + plain.rms_norm(out.double(), w.double(), 1e-5)
    assert (on_dev.cpu().double() - want).abs().max() < 1e-5
    if rounded is not None:
        assert torch.equal(rounded.cpu(), on_dev.cpu().to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,blocks,cuts", [(4, 3, [1, 2, 1, 9, 3, 30]), (2, 1, [5, 1, 1]), (3, 2, [46]), (1, 4, [3, 2])])
def test_convolution_gates_and_recurrence_across_cuts(dtype, taps, blocks, cuts):
    """A sequence fed in portions shorter and longer than the convolution, in a slot between two others: every portion's
    rows equal the plain whole-sequence values, the state carries over, and the neighbours' slots stay untouched."""

    from llm_runtime_study_b200.ops import grouped as G
    from llm_runtime_study_b200.ops import mixer_steps as M
    from llm_runtime_study_b200.ops import sequence_state as S

    torch.manual_seed(taps)
    bw = 8
    width, n = blocks * bw, sum(cuts)
    proj = torch.randn(n, 2 * width + 3).to(dtype)
    w, cb = torch.randn(width, taps), torch.randn(width)
    ra, ri = torch.randn(blocks, bw, bw).to(dtype), torch.randn(blocks, bw, bw).to(dtype)
    rab, rib, lam = torch.randn(blocks, bw), torch.randn(blocks, bw), torch.randn(width)
    gate_w = torch.cat([ra, ri], dim=1).contiguous()
    gate_b = torch.cat([rab, rib], dim=1).contiguous()
    conv_state = torch.zeros(3, max(taps - 1, 0), width, device=DEV)
    state = torch.zeros(3, width, device=DEV)
    slot = torch.tensor([1], dtype=torch.int32, device=DEV)
    outs, at = [], 0
    for m in cuts:
        part = dev(proj[at:at + m].contiguous())
        q_start = torch.tensor([0, m], dtype=torch.int32, device=DEV)
        entry = torch.zeros(m, dtype=torch.int32, device=DEV)
        u = M.conv_taps(part, dev(w), dev(cb), conv_state if taps > 1 else None, q_start=q_start, slots=slot, token_entry=entry)
        if taps > 1:
            S.conv_state_update(part, conv_state, q_start, slot)
        gates = G.batched_linear(u, dev(gate_w), batch=blocks, k=bw, n_out=2 * bw, a_batch_stride=bw, bias=dev(gate_b), out_dtype=torch.float32)
        outs.append(M.gated_recurrence(gates.view(m, blocks, 2 * bw), u, part, y_offset=width, lam=dev(lam), decay_scale=8.0,
                                       state=state, q_start=q_start, slots=slot, block_width=bw).cpu())
        at += m
    got = torch.cat(outs).double()
    x = proj.double()
    store = plain.round_bfloat16 if dtype == torch.bfloat16 else plain.keep
    u = store(plain.causal_conv(x[:, :width], w.double(), cb.double()))
    ub = u.view(n, blocks, bw)
    r = plain.sigmoid(torch.einsum("tbi,boi->tbo", ub, ra.double()) + rab.double()).reshape(n, width)
    i = plain.sigmoid(torch.einsum("tbi,boi->tbo", ub, ri.double()) + rib.double()).reshape(n, width)
    a = torch.exp(-8.0 * r * plain.softplus(lam.double()))
    s, want = torch.zeros(width, dtype=torch.float64), []
    for t in range(n):
        s = a[t] * s + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
        want.append(s * plain.gelu_tanh(x[t, width : 2 * width]))
    want = torch.stack(want)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (got - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
    assert (state[1].cpu().double() - s).abs().max() <= 1e-4 and state[0].abs().max() == 0 and state[2].abs().max() == 0
    if taps > 1:
        assert conv_state[0].abs().max() == 0 and conv_state[2].abs().max() == 0
        assert torch.equal(conv_state[1].cpu(), proj[n - (taps - 1):, :width].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,ff,experts,top", [(70, 48, 40, 5, 2), (3, 64, 24, 3, 3), (200, 32, 16, 7, 1), (1, 40, 72, 12, 3),
                                                    (700, 64, 48, 5, 2), (300, 128, 320, 3, 2)])
def test_router_and_experts_against_plain(dtype, n, width, ff, experts, top):
    """The last two cases bring enough rows for the tiles of 128 rows an expert that the tcgen05 kernel takes (bfloat16)."""

    from llm_runtime_study_b200.ops import grouped as G

    torch.manual_seed(n)
    h = torch.randn(n, width).to(dtype)
    router, rb = torch.randn(experts, width), torch.randn(experts)
    up, down = (0.3 * torch.randn(experts, ff, width)).to(dtype), (0.3 * torch.randn(experts, width, ff)).to(dtype)
    wide = G.wide_tiles_pay(n, top, dtype, width, ff)
    assert wide == (dtype == torch.bfloat16 and n * top >= 512)
    routing = G.route(dev(h), dev(router), dev(rb), top=top, wide_tiles=wide)
    z = h.double() @ router.double().T + rb.double()
    chosen = torch.topk(z, top, dim=-1)
    assert torch.equal(routing.ids.cpu().long(), chosen.indices)
    assert (routing.weights.cpu().double() - torch.softmax(chosen.values, dim=-1)).abs().max() < 1e-5
    hidden = G.expert_linear(dev(h), dev(up), routing, gather=True, act="relu2")
    rows = G.expert_linear(hidden, dev(down), routing, gather=False, out_dtype=torch.float32)
    got = G.combine(rows, routing).cpu().double()
    weights = {"router": router, "router.b": rb}
    for e in range(experts):
        weights[f"e{e}.up"], weights[f"e{e}.down"] = up[e], down[e]
    store = plain.round_bfloat16 if dtype == torch.bfloat16 else plain.keep
    want = plain.moe(h.double(), {k: v.double() for k, v in weights.items()}, {"router": {"experts": experts, "top": top}}, store)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert (got - want).abs().max() <= tol * max(1.0, float(want.abs().max()))
    # the norm behind the experts forms the weighted sum itself when it is handed the rows in pieces
    from llm_runtime_study_b200.ops import mixer_steps as M

    resid, w = torch.randn(n, width), 1 + 0.1 * torch.randn(width)
    on_dev = dev(resid.clone())
    M.norm_accumulate_round(M.PairedRows(rows, routing.pair_row, routing.weights), dev(w), 1e-5, on_dev, None)
    want_resid = resid.double() + plain.rms_norm(got, w.double(), 1e-5)
    assert (on_dev.cpu().double() - want_resid).abs().max() < 2e-5 * max(1.0, float(want_resid.abs().max()))
    # the sorted order: every pair has a row of its expert's tiles, padding rows belong to nobody
    tile = routing.tile_rows
    sorted_token, pair_row, tile_group = routing.sorted_token.cpu(), routing.pair_row.cpu(), routing.tile_group.cpu()
    assert sorted(pair_row.tolist()) == sorted((sorted_token >= 0).nonzero().flatten().tolist())
    for p, row in enumerate(pair_row.tolist()):
        assert sorted_token[row] == p // top and tile_group[row // tile] == routing.ids.cpu().flatten()[p]


def test_batched_products_with_strides():
    from llm_runtime_study_b200.ops import grouped as G

    torch.manual_seed(2)
    m, heads, k, n_out = 37, 3, 20, 12
    a = torch.randn(m, heads * 25 + 2)
    w = torch.randn(heads, n_out, k)
    bias = torch.randn(heads, n_out)
    out = torch.zeros(m, heads * 16, device=DEV)
    G.batched_linear(dev(a), dev(w), batch=heads, k=k, n_out=n_out, a_batch_stride=25, bias=dev(bias), out=out, out_batch_stride=16)
    for h in range(heads):
        want = a[:, h * 25 : h * 25 + k].double() @ w[h].double().T + bias[h].double()
        assert (out[:, h * 16 : h * 16 + n_out].cpu().double() - want).abs().max() < 1e-4
        assert out[:, h * 16 + n_out : (h + 1) * 16].abs().max() == 0
    got = G.batched_linear(dev(a), dev(w.transpose(1, 2).contiguous()), batch=heads, k=k, n_out=n_out, a_batch_stride=25, weight_k_major=True)
    for h in range(heads):
        assert (got[:, h * n_out : (h + 1) * n_out].cpu().double() - a[:, h * 25 : h * 25 + k].double() @ w[h].double().T).abs().max() < 1e-4
    # bfloat16 on the tensor cores (strides of whole 16-byte chunks) and on the CUDA cores (an odd stride)
    for stride, kk in ((32, 24), (25, 20)):
        ab = torch.randn(m, heads * stride).bfloat16()
        wb = torch.randn(heads, n_out, kk).bfloat16()
        got = G.batched_linear(dev(ab), dev(wb), batch=heads, k=kk, n_out=n_out, a_batch_stride=stride, out_dtype=torch.float32)
        for h in range(heads):
            want = ab[:, h * stride : h * stride + kk].double() @ wb[h].double().T
            assert (got[:, h * n_out : (h + 1) * n_out].cpu().double() - want).abs().max() < 1e-3 * float(want.abs().max())
    # a row's bits do not depend on its company
    alone = G.batched_linear(dev(a[5:6].contiguous()), dev(w), batch=heads, k=k, n_out=n_out, a_batch_stride=25)
    among = G.batched_linear(dev(a), dev(w), batch=heads, k=k, n_out=n_out, a_batch_stride=25)
    assert torch.equal(alone[0], among[5])


# ------------------------------------------------------------------------------------------- whole models
LENGTHS = {"A": [1, 2, 5, 23, 64, 65, 131], "B": [3, 17, 48, 70, 1, 129], "C": [140, 2, 37, 66, 300], "D": [200, 33, 40, 1, 90]}


def _requests(name):
    config, seed, _ = helpers.ROPULIX[name]
    rng = random.Random(seed + 1)
    return {f"r{i}": helpers.random_tokens(rng, config["vocab"], n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B") for d in ("float32", "bfloat16")] + [("C", "bfloat16"), ("D", "bfloat16"), ("D", "float32")], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    from llm_runtime_study_b200.engine.runtime import load

    name, dtype = request.param
    config, seed, page = helpers.ROPULIX[name]
    path, weights = helpers.make_ropulix_dir(tmp_path_factory.mktemp(f"ropulix{name}{dtype}"), config, seed, torch_dtype=dtype)
    requests = _requests(name)
    store = plain.round_bfloat16 if dtype == "bfloat16" else plain.keep
    expected, clear = {}, {}
    for rid, tokens in requests.items():
        margins = []
        expected[rid] = plain.forward(config, weights, tokens, store=store, margins=margins)
        clear[rid] = torch.stack(margins).min(dim=0).values > CLOSE_CALL if margins else torch.ones(len(tokens), dtype=torch.bool)
    loaded = load(path, device=DEV, dtype=dtype, strict_dtype=False)
    return dict(name=name, dtype=dtype, config=config, page=page, path=path, requests=requests, plain=expected, loaded=loaded,
                weights=weights, clear=clear)


def _replay(setup, steps, *, max_requests=4, max_tokens=None):
    from llm_runtime_study_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(setup["loaded"], max_tokens=max_tokens or helpers.pool_tokens(steps), page_size=setup["page"],
                             max_requests=max_requests)
    outputs = {}
    for record in steps:
        rows = replayer.run_step(record)
        if rows is not None:
            outputs[record["step"]] = torch.from_numpy(np.array(rows))
    manager = replayer.runner.manager
    manager.check()
    assert manager.active_sequences == 0 and manager.all_free and manager.free_slots == max_requests
    return helpers.collect_logits(steps, outputs)


def _compare(setup, got, requests=None):
    for rid, tokens in (requests or setup["requests"]).items():
        assert sorted(got[rid]) == list(range(len(tokens))), rid
        rows = torch.stack([got[rid][p] for p in range(len(tokens))]).double()
        if setup["dtype"] == "bfloat16":
            want = setup["plain"][rid]
            err = (rows - want).pow(2).mean(dim=1).sqrt() / want.pow(2).mean(dim=1).sqrt()
            assert torch.isfinite(err).all()
            clear = setup["clear"][rid]
            assert int(clear.sum()) >= len(tokens) // 2, "the weights make too many close calls for this test to compare anything"
            err = torch.where(clear, err, torch.zeros_like(err))
            assert float(err.max()) <= BF16_WORST, (rid, int(err.argmax()), float(err.max()))
            over = int((err > BF16_USUAL).sum())
            assert over <= max(1, len(tokens) // 10), f"request {rid}: {over} of {len(tokens)} rows beyond {BF16_USUAL}: {err}"
            continue
        bad, err, top = helpers.first_wrong_row(rows, setup["plain"][rid], TOL[setup["dtype"]])
        assert bad is None, f"request {rid}: first wrong position {bad} of {len(tokens)}, rms and largest |diff| / rms {err:.3e}, {top:.3e}"


def test_whole_prompts(setup):
    _compare(setup, _replay(setup, helpers.trace_whole(setup["requests"])))


def test_prefill_then_token_by_token(setup):
    """The tail is longer than every window, so windows pass over decoded tokens and pages behind them are given back."""

    _compare(setup, _replay(setup, helpers.trace_decode_tail(setup["requests"], tail=40)))


def test_portions_down_to_two_tokens(setup):
    rng = random.Random(5)
    _compare(setup, _replay(setup, helpers.trace_chunked(setup["requests"], rng, sizes=(2, 3, 2, 7, 13, 16, 17, 31))))


def test_mixed_batches_with_slots_and_pages_used_again(setup):
    """Three slots for seven requests, portions beside single tokens, and a pool sized for what is live."""

    rng = random.Random(9)
    steps = helpers.trace_mixed(setup["requests"], rng, live_max=3, tail=6)
    _compare(setup, _replay(setup, steps, max_requests=3))


def test_every_token_decoded_alone(setup):
    """A sequence fed one token a step from its first token: the first tokens, long decoding."""

    requests = {rid: tokens for rid, tokens in setup["requests"].items() if len(tokens) in (23, 131, 70, 66, 90)}
    _compare(setup, _replay(setup, helpers.trace_decode_tail(requests, tail=10_000)), requests)


def test_a_cut_changes_no_bit_in_float32(setup):
    if setup["dtype"] != "float32":
        pytest.skip("the 32-bit path is the one whose sums have an order fixed by the position")
    whole = _replay(setup, helpers.trace_whole(setup["requests"]))
    cut = _replay(setup, helpers.trace_chunked(setup["requests"], random.Random(1), sizes=(2, 5, 9)))
    for rid, rows in whole.items():
        for p, row in rows.items():
            assert torch.equal(row, cut[rid][p]), (rid, p)


def test_a_reused_slot_starts_from_zero(setup):
    """One slot: the second request takes the first one's state rows, convolution inputs and pages."""

    requests = {rid: tokens for rid, tokens in setup["requests"].items() if len(tokens) in (23, 17, 48, 65, 37, 66, 33, 90)}
    _compare(setup, _replay(setup, helpers.trace_chunked(requests, random.Random(3), sizes=(7, 16)), max_requests=1), requests)


def test_greedy_generation_through_the_engine(setup):
    """``Engine.generate`` with its scheduler (prompt portions, batching, graph decode where the model allows) gives the
    plain model's greedy tokens."""

    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.sampling import SamplingConfig

    if setup["dtype"] != "float32":
        pytest.skip("greedy ties are decided by rounding in bfloat16")
    config, weights = setup["config"], setup["weights"]
    prompts = [setup["requests"]["r3"][:19], setup["requests"]["r2"], setup["requests"]["r1"] + [3, 1, 4]]
    new = 12
    want = []
    for prompt in prompts:
        tokens = list(prompt)
        for _ in range(new):
            tokens.append(int(plain.forward(config, weights, tokens)[-1].argmax()))
        want.append(tokens[len(prompt):])
    engine = Engine.from_model_dir(setup["path"], device=DEV, dtype="float32", max_seq_len=64, max_batch_size=2, page_size=setup["page"],
                                   max_tokens_per_step=16, strict_dtype=False)
    got = [[] for _ in prompts]
    for index, event in engine.generate(prompts, max_new_tokens=new, sampling=SamplingConfig(temperature=0.0)):
        if event.token_id is not None:
            got[index].append(event.token_id)
    assert got == want


def test_command_line_and_trace_runner(tmp_path):
    """The command line writes a folder of random weights for the design and generates from it; the trace runner,
    started as a program with four request slots, replays a mixed trace on that folder."""

    import io
    import json
    import subprocess
    import sys
    from pathlib import Path

    from llm_runtime_study_b200.cli import main
    from llm_runtime_study_b200.weights import Checkpoint

    config = helpers.ROPULIX_B
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(config))
    out, err = io.StringIO(), io.StringIO()
    code = main(["--model", str(tmp_path / "m"), "--random-weights", str(config_path), "--weights-seed", "4",
                 "--prompt-ids", "5 17 3 90", "--max-new-tokens", "5", "--max-seq-len", "64", "--dtype", "float32", "--no-stream"],
                output=out, error=err)
    assert code == 0, err.getvalue()
    generated = [int(t) for t in out.getvalue().splitlines()[0].split()]
    weights = Checkpoint.from_model_dir(tmp_path / "m").get_tensors()
    tokens = [5, 17, 3, 90]
    for got in generated:
        logits = plain.forward(config, weights, tokens)[-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) < 1e-4:        # a tie: either token is right, and what follows differs
            break
        assert got == int(logits.argmax())
        tokens.append(got)
    rng = random.Random(2)
    requests = {f"q{i}": helpers.random_tokens(rng, config["vocab"], n) for i, n in enumerate([9, 30, 2, 17, 40])}
    steps = helpers.trace_mixed(requests, rng, live_max=4, tail=5)
    root = Path(__file__).resolve().parent.parent
    run = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32",
                          "--out", str(tmp_path / "out"), "--max-tokens", str(helpers.pool_tokens(steps))],
                         input=helpers.dump_trace(steps), capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [line for line in run.stdout.splitlines() if line.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outputs = {s["step"]: torch.from_numpy(np.fromfile(tmp_path / "out" / f"{s['step']}.f32", dtype="<f4").reshape(-1, config["vocab"]))
               for s in steps if any(e["want"] for e in s["entries"])}
    got = helpers.collect_logits(steps, outputs)
    for rid, toks in requests.items():
        want = plain.forward(config, weights, toks)
        rows = torch.stack([got[rid][p] for p in range(len(toks))]).double()
        bad, rms_err, top_err = helpers.first_wrong_row(rows, want, TOL["float32"])
        assert bad is None, (rid, bad, rms_err, top_err)
