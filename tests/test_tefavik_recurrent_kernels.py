"""The two gated recurrences of Tefavik alone, kernel by kernel, against the plain functions of `plain_tefavik.py`: the decay's
logarithm, the gates with their running maximum (token after token and as a scan), the walk of the state token by token and
chunk by chunk (sequences of unequal lengths, cut into steps, slots that are not in order), and the heads' norm with its gate.

Inputs are made so that a fault shows: a key hundreds of tokens back that only a channel without decay still holds, decays so
strong that a chunk's product underflows, gates far beyond their cap, a maximum that starts at 0 and not below."""

import numpy as np
import pytest
import torch

import plain_tefavik as pt
from rusty_llama_b200.kernels import ops

pytestmark = pytest.mark.gpu
F64 = torch.float64


def _i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")


def _walk(q, k, v, log_a, b, H, dim, vdim, lens, cuts, dtype, chunked, ext=False, q_scale=1.0):
    """Runs sequences (rows of q, k, v one after the other, `lens` tokens each) through the kernel in steps: `cuts` are the
    most tokens a sequence brings per step.  Slots are taken from the end.  Returns float64 [T, H, vdim (+1)]."""
    n_seqs, vcols = len(lens), vdim + (1 if ext else 0)
    state = torch.full((n_seqs + 2, H, dim, vcols), 7.0, device="cuda")
    slots = [n_seqs + 1 - s for s in range(n_seqs)]
    state[slots] = 0.0
    first = np.concatenate([[0], np.cumsum(lens)])
    out = torch.zeros(sum(lens), H * vcols, dtype=F64)
    done = [0] * n_seqs
    step_no = 0
    while any(d < n for d, n in zip(done, lens)):
        cut = cuts[min(step_no, len(cuts) - 1)]
        step_no += 1
        live = [s for s in range(n_seqs) if done[s] < lens[s]]
        take = [min(cut, lens[s] - done[s]) for s in live]
        rows = np.concatenate([np.arange(first[s] + done[s], first[s] + done[s] + n) for s, n in zip(live, take)])
        proj = torch.cat([q[rows], k[rows], v[rows]], dim=1).to("cuda", dtype).contiguous()
        qs, ks, vs = proj[:, : H * dim], proj[:, H * dim: 2 * H * dim], proj[:, 2 * H * dim:]
        la = log_a[rows].to("cuda", torch.float32).contiguous()
        bb = None if b is None else b[rows].to("cuda", torch.float32).contiguous()
        start = _i32(np.concatenate([[0], np.cumsum(take)]))
        ids = _i32([slots[s] for s in live])
        if chunked:
            scratch = torch.empty(ops.gated_attn_chunked_scratch_floats(len(live), max(take), H, dim, vcols), device="cuda")
            o = ops.gated_attn_chunked(qs, ks, vs, la, bb, state, ids, start, H, dim, vdim, max(take), scratch, q_scale=q_scale, ext=ext)
        else:
            o = ops.gated_attn(qs, ks, vs, la, bb, state, ids, start, H, dim, vdim, q_scale=q_scale, ext=ext)
        out[rows] = o.to(F64).cpu()
        for s, n in zip(live, take):
            done[s] += n
    assert bool((state[[0, 1]] == 7.0).all()), "a slot that no sequence owns was written"
    return out.view(sum(lens), H, vcols)


def _plain_gla(q, k, v, log_a, H, dim, vdim, lens):
    outs, at = [], 0
    for n in lens:
        s = slice(at, at + n)
        outs.append(pt.gla_recurrence(q[s].view(n, H, dim), k[s].view(n, H, dim), v[s].view(n, H, vdim), torch.exp(log_a[s]).view(n, H, dim)))
        at += n
    return torch.cat(outs)


def _inputs(T, H, dim, vdim, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(T, H * n, generator=g, dtype=F64).to(dtype).to(F64) for n in (dim, dim, vdim))
    return q, k, v, g


def test_log_decay_against_the_plain_formula():
    g = torch.Generator().manual_seed(1)
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-6)):
        z = (6 * torch.randn(37, 3 * 20, generator=g)).to(dtype)
        bias = torch.randn(60, generator=g)
        got = ops.gla_log_decay(z.cuda()[:, :60], bias.cuda(), 7.0).to(F64).cpu()
        want = pt.log_logistic(z.to(F64) + bias.to(F64)) / 7.0
        assert float((got - want).abs().max()) <= tol * (1 + float(want.abs().max()))


@pytest.mark.parametrize("H, dim, vdim", [(3, 24, 40), (2, 16, 67), (1, 8, 132)])  # (one column tile; a tile and three columns; two and four)
@pytest.mark.parametrize("chunked", [False, True])
def test_gated_linear_attention_in_steps(chunked, H, dim, vdim):
    lens = [150, 1, 67, 64]
    dtype = torch.bfloat16 if chunked else torch.float32
    q, k, v, g = _inputs(sum(lens), H, dim, vdim, 2, dtype)
    log_a = -torch.rand(sum(lens), H * dim, generator=g, dtype=F64) * 0.2
    want = _plain_gla(q, k, v, log_a.float().to(F64), H, dim, vdim, lens)
    for cuts in ([200], [64, 33, 2], [70, 1, 1, 40]):
        got = _walk(q, k, v, log_a, None, H, dim, vdim, lens, cuts, dtype, chunked and cuts[0] >= 32)
        assert float((got - want).abs().max()) <= (5e-5 if chunked else 2e-5) * float(want.abs().max()), cuts


@pytest.mark.parametrize("chunked", [False, True])
def test_a_key_hundreds_of_tokens_back_and_decays_that_underflow(chunked):
    """Channel 0 never decays and holds token 2's key; every other channel decays by e^-3 a token (e^-192 over a chunk)."""
    H, dim, vdim, T = 2, 16, 72, 333
    dtype = torch.bfloat16 if chunked else torch.float32
    q, k, v, g = _inputs(T, H, dim, vdim, 3, dtype)
    k.view(T, H, dim)[:, :, 0] = 0.0
    k.view(T, H, dim)[2, :, 0] = 8.0
    q.view(T, H, dim)[:, :, 0] = 0.0
    q.view(T, H, dim)[T - 1, :, 0] = 4.0
    log_a = torch.full((T, H, dim), -3.0, dtype=F64)
    log_a[:, :, 0] = 0.0
    log_a = log_a.view(T, H * dim)
    want = _plain_gla(q, k, v, log_a, H, dim, vdim, [T])
    far = 32.0 * v.view(T, H, vdim)[2]
    assert float((want[T - 1] - far).abs().max()) < 0.5 * float(far.abs().max())  # the last token reads token 2's values back
    for cuts in ([T], [300, 1]):
        got = _walk(q, k, v, log_a, None, H, dim, vdim, [T], cuts, dtype, chunked)
        assert torch.isfinite(got).all()
        assert float((got - want).abs().max()) <= (5e-5 if chunked else 2e-5) * float(want.abs().max())


def _plain_gates(gi, gf, bi, bf, cap, lens):
    """log_a, b, m per token as the recurrence takes them, the maximum starting at 0 in every sequence."""
    li = pt.capped(gi + bi, cap)
    lf = pt.log_logistic(pt.capped(gf + bf, cap))
    la, b, m = torch.zeros_like(li), torch.zeros_like(li), torch.zeros_like(li)
    at = 0
    for n in lens:
        mm = torch.zeros(gi.shape[1], dtype=F64)
        for t in range(at, at + n):
            m_new = torch.maximum(lf[t] + mm, li[t])
            la[t], b[t], m[t] = lf[t] + mm - m_new, torch.exp(li[t] - m_new), m_new
            mm = m_new
        at += n
    return li, lf, la, b, m


@pytest.mark.parametrize("scan", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gates_and_running_maximum(scan, dtype):
    H, cap, lens = 5, 6.0, [700, 3, 257, 256]
    g = torch.Generator().manual_seed(4)
    T = sum(lens)
    raw = (9 * torch.randn(T, 2 * H + 3, generator=g)).to(dtype)  # far beyond the cap on both sides
    raw[:40, 3: 3 + H] = -30.0  # input gates at the cap's lower end when a sequence starts: the first maxima come from the start value 0
    bi, bf = torch.randn(H, generator=g), torch.randn(H, generator=g)
    gi, gf = raw.to(F64)[:, 3: 3 + H], raw.to(F64)[:, 3 + H:]
    li_w, _, la_w, b_w, m_w = _plain_gates(gi, gf, bi.to(F64), bf.to(F64), cap, lens)
    assert float((m_w[0] - li_w[0]).max()) > 0.1  # a maximum that started at minus infinity would be the input gate itself
    dev = raw.cuda()
    for cuts in ([1000], [256, 300, 1, 1]):
        m_state = torch.full((len(lens) + 1, H), 5.0, device="cuda")
        m_state[1:] = 0.0
        first, done = np.concatenate([[0], np.cumsum(lens)]), [0] * len(lens)
        la_g, b_g, m_g = (torch.zeros(T, H, dtype=F64) for _ in range(3))
        for cut in cuts + [10 ** 6]:
            live = [s for s in range(len(lens)) if done[s] < lens[s]]
            if not live:
                break
            take = [min(cut, lens[s] - done[s]) for s in live]
            rows = np.concatenate([np.arange(first[s] + done[s], first[s] + done[s] + n) for s, n in zip(live, take)])
            part = dev[torch.as_tensor(rows, device="cuda")].contiguous()
            la, b, m = ops.mlstm_gates(part[:, 3: 3 + H], part[:, 3 + H:], bi.cuda(), bf.cuda(), cap, m_state, _i32([s + 1 for s in live]),
                                       _i32(np.concatenate([[0], np.cumsum(take)])), scan=scan)
            la_g[rows], b_g[rows], m_g[rows] = la.to(F64).cpu(), b.to(F64).cpu(), m.to(F64).cpu()
            for s, n in zip(live, take):
                done[s] += n
        assert bool((m_state[0] == 5.0).all())
        last = torch.as_tensor(first[1:] - 1)
        assert float((m_state[1:].to(F64).cpu() - m_w[last]).abs().max()) <= 2e-5
        for got, want in ((la_g, la_w), (b_g, b_w), (m_g, m_w)):
            assert float((got - want).abs().max()) <= 3e-5, (scan, cuts)


@pytest.mark.parametrize("chunked", [False, True])
def test_matrix_memory_with_its_normaliser(chunked):
    H, dim, vdim, cap, lens = 2, 32, 64, 8.0, [130, 45]
    dtype = torch.bfloat16 if chunked else torch.float32
    T = sum(lens)
    q, k, v, g = _inputs(T, H, dim, vdim, 5, dtype)
    gi, gf = 4 * torch.randn(T, H, generator=g, dtype=F64), 4 * torch.randn(T, H, generator=g, dtype=F64) + 2
    zero = torch.zeros(H, dtype=F64)
    li, lf, la, b, m = _plain_gates(gi, gf, zero, zero, cap, lens)
    want, at = [], 0
    for n in lens:
        s = slice(at, at + n)
        want.append(pt.mlstm_recurrence(q[s].view(n, H, dim) * dim ** -0.5, k[s].view(n, H, dim), v[s].view(n, H, vdim), li[s], lf[s]))
        at += n
    want = torch.cat(want)
    weight = torch.rand(H * vdim, generator=g) + 0.5
    gate = torch.randn(T, H * vdim, generator=g).to(dtype)
    want_y = pt.rms(want, 1e-5).reshape(T, H * vdim) * weight.to(F64) * pt.logistic(gate.to(F64))
    for cuts in ([200], [64, 40, 2]):
        o = _walk(q, k, v, la, b, H, dim, vdim, lens, cuts, dtype, chunked and cuts[0] >= 32, ext=True, q_scale=dim ** -0.5)
        den = torch.maximum(o[:, :, vdim].abs(), torch.exp(-m)) + 1e-6
        got = o[:, :, :vdim] / den[:, :, None]
        assert float((got - want).abs().max()) <= 5e-5 * float(want.abs().max()), cuts
        y = ops.head_norm_gate(o.reshape(T, -1).float().cuda(), H, vdim, weight.cuda(), 1e-5, gate.cuda(), ops.GATE_SIGMOID, dtype,
                               m=m.float().cuda(), den_eps=1e-6)
        tol = 2e-5 if dtype == torch.float32 else 1e-2
        assert float((y.to(F64).cpu() - want_y).abs().max()) <= tol * float(want_y.abs().max())


def test_heads_norm_with_a_shared_weight_and_silu():
    g = torch.Generator().manual_seed(6)
    T, H, n = 9, 3, 40
    x = torch.randn(T, H * n, generator=g)
    w = torch.rand(n, generator=g) + 0.5
    gate = torch.randn(T, H * n, generator=g)
    y = ops.head_norm_gate(x.cuda(), H, n, w.cuda(), 1e-4, gate.cuda(), ops.GATE_SILU, torch.float32, out_scale=0.5)
    gg = gate.to(F64)
    want = pt.rms_norm(x.to(F64).view(T, H, n), w.to(F64), 1e-4).reshape(T, H * n) * gg * pt.logistic(gg) * 0.5
    assert float((y.to(F64).cpu() - want).abs().max()) <= 1e-5
