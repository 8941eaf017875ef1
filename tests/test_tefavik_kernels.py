"""Tefavik's mechanisms alone, kernel by kernel, with inputs made so that a fault shows: one key at a chunk's first place
(or the one before it) that fits the query, keys that are all zero so that only the sink shares the probability, a raw score
far above the cap, a state that must give one token back after hundreds, decays that a careless chunked form cannot hold.

Every attention kernel that can run the design's attention is driven the same way (`attend`): the general kernel in both
element types, the tensor-core kernel for unequal key and value sizes (prompts and single tokens), the tcgen05 prompt kernel
and the TMA-fed decode kernel (equal sizes of 64 and 128).  References: `plain_tefavik.py`."""

import math

import numpy as np
import pytest
import torch

import plain_tefavik as pt

pytestmark = pytest.mark.gpu
F64 = torch.float64


def _dev(a, dtype):
    return torch.as_tensor(np.asarray(a, dtype=np.float64)).to("cuda", dtype)


def _rounded(a, dtype):
    return _dev(a, dtype).to(F64).cpu().numpy()


def _i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")


def _paged(k, v, dtype, n_pages, order):
    """k [L, G, kd], v [L, G, vd] laid into pages in the given order of page ids; unused places hold finite junk."""
    L, G, kd = k.shape
    kp = torch.full((n_pages, G, 64, kd), 4.0, dtype=dtype, device="cuda")
    vp = torch.full((n_pages, G, 64, v.shape[2]), -3.0, dtype=dtype, device="cuda")
    for i in range((L + 63) // 64):
        n = min(64, L - 64 * i)
        kp[order[i], :, :n] = _dev(k[64 * i: 64 * i + n], dtype).transpose(0, 1)
        vp[order[i], :, :n] = _dev(v[64 * i: 64 * i + n], dtype).transpose(0, 1)
    return kp, vp, order[: (L + 63) // 64]


def plain_rows(q, k, v, p0, scale, softcap, chunk):
    """The plain attention's rows for queries q [n, H, kd] at positions p0 .. p0 + n - 1 over keys k [L, G, kd], v [L, G, vd]."""
    n, H, _ = q.shape
    G = k.shape[1]
    L = p0 + n
    visible = pt.chunk_mask(L, chunk)[p0:]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = torch.as_tensor(q[:, h]) @ torch.as_tensor(k[:L, g]).T * scale
        s = softcap * torch.tanh(s / softcap)
        out.append(pt.softmax_plus_one(s, visible) @ torch.as_tensor(v[:L, g]))
    return torch.stack(out, dim=1).numpy()


KERNELS = {
    "general-32": torch.float32, "general-16": torch.bfloat16, "unequal-sizes": torch.bfloat16, "unequal-sizes-single": torch.bfloat16,
    "tcgen05-prompt": torch.bfloat16, "tma-single": torch.bfloat16, "the part's choice": torch.bfloat16,
}


def attend(kernel, q, kp, vp, pages, p0, H, G, kd, vd, scale, softcap, chunk):
    """q [n, H, kd] (already rounded) at positions p0 .. of ONE sequence whose pages are `pages` -> [n, H, vd] float64."""
    from rusty_llama_b200.kernels import ops
    from rusty_llama_b200.parts.attention import chunked_attention_runner

    dtype = KERNELS[kernel]
    n = q.shape[0]
    rows = torch.zeros((n, H * kd + 8), dtype=dtype, device="cuda")  # rows longer than the queries, as a projection's are
    rows[:, : H * kd] = _dev(q.reshape(n, H * kd), dtype)
    sink = torch.zeros(H, dtype=torch.float32, device="cuda")
    table = _i32([pages])
    single = kernel in ("unequal-sizes-single", "tma-single")
    if kernel.startswith("general"):
        out = ops.attn_ext(rows, kp, vp, table, _i32(np.zeros(n)), _i32(np.arange(p0, p0 + n)), H, G, kd, vd, scale, sink=sink, chunk=chunk, softcap=softcap)
    elif kernel == "unequal-sizes":
        out = ops.flash_mix(rows, kp, vp, table, _i32([0, n]), _i32([p0]), n, H, G, kd, vd, scale, sink=sink, chunk=chunk, softcap=softcap)
    elif kernel == "tcgen05-prompt":
        out = ops.flash_prefill_tc(rows, kp, vp, table, _i32([0, n]), _i32([p0]), n, H, G, kd, sink=sink, scale=scale, chunk=chunk, softcap=softcap)
    elif kernel == "the part's choice":
        from types import SimpleNamespace

        step = SimpleNamespace(tok_seq=_i32(np.zeros(n)), tok_pos=_i32(np.arange(p0, p0 + n)), seq_start=_i32([0, n]), seq_pos0=_i32([p0]),
                               max_q_len=n, n_seqs=1, decode_only=n == 1)
        out = chunked_attention_runner(rows, kp, vp, table, step, H, G, kd, vd, scale, chunk, softcap, sink)()
    elif single:  # every row a sequence of its own on the same pages, one token each
        tables = _i32([pages] * n)
        if kernel == "tma-single":
            splits = 2
            scratch = torch.empty(ops.attn_decode_scratch_floats(n, H, kd, splits), dtype=torch.float32, device="cuda")
            out = ops.attn_decode(rows, kp, vp, tables, _i32(np.arange(p0, p0 + n) + 1), H, G, kd, splits, scratch, scale=scale, sink=sink,
                                  chunk=chunk, softcap=softcap, impl="tma")
        else:
            splits = 3
            qf = ops.fold_queries(rows, torch.eye(H, dtype=torch.float32, device="cuda"), H, G, kd)
            scratch = torch.empty(ops.flash_mix_decode_scratch_floats(n, H, vd, splits), dtype=torch.float32, device="cuda")
            out = ops.flash_mix_decode(qf, kp, vp, tables, _i32(np.arange(p0, p0 + n)), H, G, kd, vd, scale, splits, scratch, sink=sink,
                                       chunk=chunk, softcap=softcap)
    ops.tc_status_check()
    return out.to(F64).cpu().numpy().reshape(n, H, vd)


def takes(kernel, H, G, kd, vd):
    from rusty_llama_b200.kernels import ops

    if kernel in ("tcgen05-prompt", "tma-single"):
        return kd == vd and kd in (64, 128)
    if kernel == "unequal-sizes":
        return ops.flash_mix_takes(kd, vd, 1)
    if kernel == "unequal-sizes-single":
        return ops.flash_mix_takes(kd, vd, 1) and ops.flash_mix_decode_takes(H, G, kd, vd)
    return True


SHAPES = [(6, 2, 24, 40), (4, 4, 64, 64), (2, 1, 128, 128), (8, 2, 48, 16), (1, 1, 8, 8)]


def _tol(kernel):
    return 2e-5 if KERNELS[kernel] == torch.float32 else 2e-2


@pytest.mark.parametrize("kernel", list(KERNELS))
@pytest.mark.parametrize("chunk", [1, 2, 7, 64, 65, 130, 200])
def test_chunk_edges_in_prompts_and_single_tokens(kernel, chunk):
    """The key at a chunk's first position e, and the key before it, are each made to fit all queries in turn.  Queries stand at
    e - 2 .. e + 3 and, a chunk later, at e + chunk - 2 .. e + chunk + 1: those of e's chunk must return the first key's value
    (also from far back), the others must not know it; the key before e belongs to the queries before e only.  Chunks of one
    token, of a page, of a page and one, of two pages and a bit; edges at, before and after page borders; the first tokens."""
    rng = np.random.default_rng(chunk)
    L = 64 * 5
    order = [4, 0, 5, 1, 2]
    for H, G, kd, vd in SHAPES[:3]:
        if not takes(kernel, H, G, kd, vd):
            continue
        dtype = KERNELS[kernel]
        k0 = _rounded(0.1 * rng.standard_normal((L, G, kd)), dtype)
        v = _rounded(rng.standard_normal((L, G, vd)), dtype)
        a = math.sqrt(40.0 / kd)
        edges = sorted({e for e in (chunk, (128 // chunk) * chunk, (129 // chunk + 1) * chunk, (L - 6) // chunk * chunk) if 2 <= e <= L - 4})[:4]
        for e in [0] + edges:
            for hot in (e, e - 1):
                if hot < 0:
                    continue
                k = k0.copy()
                k[hot] = _rounded(np.full((G, kd), a), dtype)
                kp, vp, pages = _paged(k, v, dtype, 6, order)
                for p0, n in ((max(e - 2, 0), 6 if e >= 2 else 4), (e + chunk - 2, 4)):
                    if p0 < 0 or p0 + n > L:
                        continue
                    q = _rounded(np.full((n, H, kd), a), dtype)
                    got = attend(kernel, q, kp, vp, pages, p0, H, G, kd, vd, 1.0, 100.0, chunk)
                    ref = plain_rows(q, k, v, p0, 1.0, 100.0, chunk)
                    assert np.abs(got - ref).max() <= _tol(kernel) * max(1.0, np.abs(ref).max()), (H, kd, e, hot, p0)
                    for r in range(n):
                        p = p0 + r
                        sees = hot <= p and hot // chunk == p // chunk
                        gap = np.abs(got[r, 0] - v[hot, 0]).max()
                        assert (gap < 0.03) if sees else (gap > 0.2), (H, kd, e, hot, p, gap)


@pytest.mark.parametrize("kernel", list(KERNELS))
def test_the_sink_takes_its_share_and_the_cap_holds(kernel):
    """All keys zero: the n keys a query sees and the sink share the probability equally, so the result is n / (n + 1) of
    the mean of the values of its chunk so far.  Then one key whose raw score is 1000: under a cap of 3 it may take
    e^3 / (1 + e^3 + n - 1) and no more."""
    rng = np.random.default_rng(3)
    L, chunk = 150, 70
    for H, G, kd, vd in SHAPES:
        if not takes(kernel, H, G, kd, vd):
            continue
        dtype = KERNELS[kernel]
        v = _rounded(rng.standard_normal((L, G, vd)), dtype)
        k = np.zeros((L, G, kd))
        kp, vp, pages = _paged(k, v, dtype, 4, [2, 0, 3])
        p0, n = 136, 6  # crosses the edge at 140
        q = _rounded(rng.standard_normal((n, H, kd)), dtype)
        got = attend(kernel, q, kp, vp, pages, p0, H, G, kd, vd, 0.5, 7.0, chunk)
        for r in range(n):
            p = p0 + r
            lo = p - p % chunk
            share = (p - lo + 1) / (p - lo + 2)
            want = share * v[lo: p + 1].mean(axis=0)  # [G, vd]
            for h in range(H):
                assert np.abs(got[r, h] - want[h // (H // G)]).max() <= 1e-5 + _tol(kernel) / 2, (H, kd, p, h)
        a = math.sqrt(1000.0 / kd)
        k[143] = np.full((G, kd), a)
        k = _rounded(k, dtype)
        kp, vp, pages = _paged(k, v, dtype, 4, [2, 0, 3])
        q = _rounded(np.full((n, H, kd), a), dtype)
        got = attend(kernel, q, kp, vp, pages, p0, H, G, kd, vd, 1.0, 3.0, chunk)
        ref = plain_rows(q, k, v, p0, 1.0, 3.0, chunk)
        assert np.abs(got - ref).max() <= _tol(kernel), (H, kd)
        seen = 146 - 140 + 1
        most = math.exp(3.0) / (1.0 + math.exp(3.0) + seen - 1)
        rest = got[n - 1, 0] - most * v[143, 0]
        assert np.abs(rest).max() > 0.01 and np.abs(got[n - 1, 0] - v[143, 0]).max() > 0.02, "the cap does not hold"


@pytest.mark.parametrize("kernel", list(KERNELS))
def test_random_scores_in_portions_and_alone(kernel):
    """Peaked random scores, grouped heads, a scale and a cap that both matter: a prompt whole, then the same rows as portions
    of 2, 61 and 3 tokens and one by one over the cache, against the plain rows."""
    rng = np.random.default_rng(11)
    L = 200
    for (H, G, kd, vd), chunk, cap, scale in zip(SHAPES, (50, 64, 130, 33, 3), (4.0, 30.0, 8.0, 2.0, 50.0), (0.7, 0.125, 0.2, 0.4, 1.0)):
        if not takes(kernel, H, G, kd, vd):
            continue
        dtype = KERNELS[kernel]
        k = _rounded(rng.standard_normal((L, G, kd)), dtype)
        v = _rounded(rng.standard_normal((L, G, vd)), dtype)
        q = _rounded(1.5 * rng.standard_normal((L, H, kd)), dtype)
        kp, vp, pages = _paged(k, v, dtype, 5, [1, 4, 0, 2])
        ref = plain_rows(q, k, v, 0, scale, cap, chunk)
        single = kernel.endswith("single")
        cuts = [(0, 5), (62, 4), (126, 5), (195, 5)] if single else [(0, L), (0, 2), (2, 61), (63, 3), (66, 1), (127, 2), (129, 71)]
        for p0, n in cuts:
            got = attend(kernel, q[p0: p0 + n], kp, vp, pages, p0, H, G, kd, vd, scale, cap, chunk)
            assert np.abs(got - ref[p0: p0 + n]).max() <= _tol(kernel) * max(1.0, np.abs(ref).max()), (H, kd, p0, n)


@pytest.mark.parametrize("dtype, H, G, kd, vd, rot, pad", [
    (torch.bfloat16, 4, 2, 64, 32, 32, 0),     # rows of 16 bytes: eight numbers to a thread, a head's threads add up by shuffles
    (torch.bfloat16, 3, 1, 128, 128, 128, 8),  # 16 threads to a head; more heads than fill the block's first round evenly
    (torch.bfloat16, 40, 8, 8, 8, 0, 0),       # one thread to a head, no rotation, two rounds of the block
    (torch.bfloat16, 2, 2, 16, 24, 8, 3),      # a row stride that is no multiple of 8: the element-wise kernel
    (torch.float32, 4, 2, 64, 32, 32, 0),
    (torch.float32, 3, 1, 20, 12, 6, 1),
])
def test_biases_norms_of_heads_rotation_and_cache_write(dtype, H, G, kd, vd, rot, pad):
    """q in place, k and v in shuffled pages, positions around a page border, weights of the norms that differ from 1."""
    g = torch.Generator().manual_seed(kd + vd)
    pos = torch.tensor([62, 63, 64, 65, 0, 1, 700])
    seq = [0, 0, 0, 0, 1, 1, 2]
    T, cols, eps, base = len(seq), (H + G) * kd + G * vd, 1e-3, 300.0
    x = torch.randn(T, cols + pad, generator=g, dtype=F64).to(dtype).to(F64)
    bias = torch.randn(cols, generator=g).to(F64)
    wq, wk = (torch.rand(kd, generator=g) + 0.5).to(F64), (torch.rand(kd, generator=g) + 0.5).to(F64)
    freq = (base ** (-2.0 * torch.arange(rot // 2, dtype=F64) / max(rot, 1))).float()
    table = _i32([[3, 1] + [0] * 9, [2, 0] + [0] * 9, [5] * 10 + [4]])
    kp = torch.zeros((6, G, 64, kd), dtype=dtype, device="cuda")
    vp = torch.zeros((6, G, 64, vd), dtype=dtype, device="cuda")
    xt = x.to("cuda", dtype)
    from rusty_llama_b200.kernels import ops
    ops.qkv_prep(xt, bias.float().cuda(), _i32(pos.numpy()), _i32(seq), table, kp, vp, freq.cuda() if rot else None, 1.0, H, G, kd, vd, rot, True,
                 q_norm=wq.float().cuda(), k_norm=wk.float().cuda(), norm_eps=eps)
    y = x[:, :cols] + bias

    def plain(heads, w):  # the frequencies as the kernel gets them, rounded to 32 bits
        heads = pt.rms_norm(heads, w, eps)
        if not rot:
            return heads
        ang = pos.to(F64)[:, None] * freq.to(F64)[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = heads.clone()
        u, w2 = heads[..., 0:rot:2], heads[..., 1:rot:2]
        out[..., 0:rot:2], out[..., 1:rot:2] = u * c - w2 * s, w2 * c + u * s
        return out

    q_ref = plain(y[:, : H * kd].reshape(T, H, kd), wq)
    k_ref = plain(y[:, H * kd: (H + G) * kd].reshape(T, G, kd), wk)
    v_ref = y[:, (H + G) * kd:].reshape(T, G, vd)
    tol = 3e-5 if dtype == torch.float32 else 3e-2  # (position 700 times a 32-bit frequency: the angle itself carries 4e-5)
    got = xt.to(F64).cpu()
    assert float((got[:, : H * kd].reshape(T, H, kd) - q_ref).abs().max()) <= tol * 4
    assert torch.equal(got[:, cols:], x[:, cols:])
    tab = table.cpu()
    for t in range(T):
        page = int(tab[seq[t], int(pos[t]) // 64])
        assert float((kp[page, :, int(pos[t]) % 64].to(F64).cpu() - k_ref[t]).abs().max()) <= tol * 4, t
        assert float((vp[page, :, int(pos[t]) % 64].to(F64).cpu() - v_ref[t]).abs().max()) <= tol, t
    used = {int(tab[s, int(p) // 64]) for s, p in zip(seq, pos)}
    for page in set(range(6)) - used:
        assert not bool(kp[page].any()) and not bool(vp[page].any())
