"""Namalix beside Revirax (the library's closest model: a linear attention with a constant decay per head, which is the
retention layer's recurrence, an attention whose heads are mixed and gated, dense feed-forwards) at equal sizes: prompt-step
and decode-step throughput through the engine, and every kernel that only Namalix uses timed alone beside the kernel of
Revirax or Llama that does the like work.

    python bench.py --design namalix [--design-sizes small,lite,wide]

Sizes resemble real models' layers (random weights, four layers: attention, retention, delta, attention; the whole vocabulary;
dense feed-forwards in the first and third layer, experts in the other two).  Revirax beside it has the same width, heads,
kv heads, head size, layer count and vocabulary, a window that never binds at these lengths, and a dense feed-forward with as
many weights as the experts that a token of Namalix uses.  Every kernel's fraction is what it must move (bytes, against the
measured copy rate) or compute (flops, against the measured bfloat16 matrix rate), whichever bound is the tighter one,
divided by the time it took.
"""

from __future__ import annotations

import math
from types import SimpleNamespace
from typing import Dict

import torch

from . import microbench as mb
from . import ops
from .design_bench import _frac, step_times
from .tefavik_bench import revirax_config

SIZES = {
    "small": dict(width=1024, heads=8, kv_heads=2, hd=128, experts=8, top=2, eff=1408, vocab=32000),
    "lite": dict(width=2048, heads=16, kv_heads=4, hd=128, experts=16, top=2, eff=2816, vocab=32000),
    "wide": dict(width=4096, heads=32, kv_heads=8, hd=128, experts=16, top=2, eff=4096, vocab=32000),
}
LAYERS = 4
TAPS = 4


def namalix_config(z: dict) -> dict:
    H, G, hd = z["heads"], z["kv_heads"], z["hd"]
    attn = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": 1.0 / math.sqrt(hd), "softcap": 30.0, "v_mix": True,
            "rot": {"base": 10000.0, "dims": hd // 2, "scaling": {"factor": 8.0, "original": 8192, "fast": 16.0, "slow": 2.0}}}
    ret = {"heads": H, "dim": hd, "vdim": hd, "decay": [1.0 - 2.0 ** (-3 - 5 * i / max(H - 1, 1)) for i in range(H)], "rot": {"base": 1000000.0, "dims": hd}}
    delta = {"heads": H, "kv_heads": H, "dim": hd, "vdim": hd, "conv": TAPS}
    dense = {"kind": "dense", "ff": z["top"] * z["eff"]}
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"], "scale": 1.5}, "expert": {"ff": z["eff"], "limit": 7.0}}
    layers = [{"type": "attention", "mixer": attn, "mlp": dense}, {"type": "retention", "mixer": ret, "mlp": moe},
              {"type": "delta", "mixer": delta, "mlp": dense}, {"type": "attention", "mixer": attn, "mlp": moe}]
    return {"architecture": "Namalix", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0}, "layers": layers}


def kernel_table(z: dict, T: int, batch: int, ctx: int, peaks: dict) -> Dict[str, dict]:
    """Each kernel of the design alone, at a prompt step of T tokens (one sequence) and a decode step of `batch` sequences at `ctx`."""
    from ..parts import attention as attention_part

    dev, bf = "cuda:0", torch.bfloat16
    H, G, hd = z["heads"], z["kv_heads"], z["hd"]
    out: Dict[str, dict] = {}
    it = dict(iters=10, warmup=2)
    scale = 1.0 / math.sqrt(hd)

    def note(name, us, nbytes, flops, like=None):
        out[name] = {"us": round(us, 1), "frac": _frac(us, nbytes, flops, peaks)}
        if like:
            out[name]["like"] = like

    like_prefill = mb.bench_flash_prefill(SimpleNamespace(tokens=T, impl="auto", heads=H, kv_heads=G, head_dim=hd, splits=0, **it))
    like_prefill = {"kernel": like_prefill["kernel"], "us": like_prefill["us"], "frac": round(like_prefill["causal_TFLOPs"] / peaks["bf16_tflops"], 3)}
    like_decode = mb.bench_attn_decode(SimpleNamespace(seqs=batch, ctx=ctx, impl="auto", heads=H, kv_heads=G, head_dim=hd, splits=0, **it))
    like_decode = {"kernel": "attn_decode", "us": like_decode["us"], "frac": round(like_decode["GBps"] / peaks["hbm_gbs"], 3)}

    for rows, n_seqs, pos0, tag in ((T, 1, 0, "prefill"), (batch, batch, ctx - 1, "decode")):
        per = rows // n_seqs
        prompt = rows > batch
        step = SimpleNamespace(
            tok_seq=torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(per),
            tok_pos=(pos0 + torch.arange(per, dtype=torch.int32, device=dev)).repeat(n_seqs),
            seq_start=torch.arange(n_seqs + 1, dtype=torch.int32, device=dev) * per,
            seq_pos0=torch.full((n_seqs,), pos0, dtype=torch.int32, device=dev),
            slot_ids=torch.arange(n_seqs, dtype=torch.int32, device=dev), max_q_len=per, n_seqs=n_seqs, decode_only=not prompt,
            plan_kv_len=pos0 + per,
        )
        # ---- attention with logistic weights: rotation, value blend and cache write; then the attention and the heads' mix
        pages = (pos0 + per + 63) // 64
        kp = torch.randn(n_seqs * pages, G, 64, hd, device=dev, dtype=bf)
        vp = torch.randn(n_seqs * pages, G, 64, hd, device=dev, dtype=bf)
        table = torch.randperm(n_seqs * pages, device=dev).to(torch.int32).view(n_seqs, pages).contiguous()
        qkv = torch.randn(rows, (H + 2 * G) * hd + H, device=dev, dtype=bf)
        first = torch.randn(rows, G * hd, device=dev, dtype=bf)
        lam = torch.full((1,), 0.4, device=dev)
        freq = torch.rand(hd // 4, device=dev)
        us = mb._time(lambda i: ops.qkv_prep(qkv, None, step.tok_pos, step.tok_seq, table, kp, vp, freq, 1.1, H, G, hd, hd, hd // 2, True,
                                             v_src=first, v_lambda=lam), 1, **it)
        us_like = mb._time(lambda i: ops.rope_kv_write(qkv, step.tok_pos, step.tok_seq, table, kp, vp, freq, H, G, hd, hd // 2, True), 1, **it)
        nbytes = rows * ((H + G) * hd * 4 + G * hd * 6)
        note(f"{tag}_rotate_blend_store", us, nbytes, 0, like={"kernel": "rope_kv_write", "us": round(us_like, 1), "frac": _frac(us_like, rows * (H + 2 * G) * hd * 4, 0, peaks)})
        pb = torch.full((H,), -4.0, device=dev)
        mix = (torch.eye(H, device=dev) + 0.1 * torch.randn(H, H, device=dev)).contiguous()
        gate = qkv[:, (H + 2 * G) * hd:]
        run = attention_part.logistic_attention_runner(qkv, gate, kp, vp, table, step, H, G, hd, hd, scale, 30.0, pb, mix)
        us = mb._time(lambda i: run(), 1, **it)
        keys = sum(range(pos0 + 1, pos0 + per + 1)) * n_seqs
        like = like_prefill if prompt else like_decode
        # Revirax's attention with mixed scores at the same sizes (folded queries, then the tensor-core kernel)
        if prompt:
            us_mixed = mb._time(lambda i: ops.flash_mix(ops.fold_queries(qkv, mix, H, G, hd), kp, vp, table, step.seq_start, step.seq_pos0, per, H, G, hd, hd,
                                                        scale, folded=True, gate=None), 1, **it)
            like = dict(like, mixed={"kernel": "fold_queries + flash_mix", "us": round(us_mixed, 1), "frac": _frac(us_mixed, 0, 4.0 * keys * H * hd, peaks)})
        note(f"{tag}_attention_logistic_mixed", us, n_seqs * (pos0 + per) * G * 2 * hd * 2 + rows * H * hd * 4, 4.0 * keys * H * hd, like=like)
        run_plain = attention_part.logistic_attention_runner(qkv, gate, kp, vp, table, step, H, G, hd, hd, scale, 30.0, pb, None)
        us = mb._time(lambda i: run_plain(), 1, **it)
        note(f"{tag}_attention_logistic_unmixed", us, n_seqs * (pos0 + per) * G * 2 * hd * 2 + rows * H * hd * 4, 4.0 * keys * H * hd, like=like_prefill if prompt else like_decode)
        # ---- retention: the rotation of q and k in place, Revirax's recurrence kernels, every head's norm and the gate
        qd = H * hd
        proj = torch.randn(rows, 4 * qd + 2 * H, device=dev, dtype=bf)
        q, k, v, g = (proj[:, i * qd: (i + 1) * qd] for i in range(4))
        freq2 = torch.rand(hd // 2, device=dev)
        us = mb._time(lambda i: ops.rope_kv_write(proj, step.tok_pos, step.tok_seq, None, None, None, freq2, 2 * H, 0, hd, hd, False, write_kv=False), 1, **it)
        note(f"{tag}_retention_rotate_q_k", us, rows * 2 * qd * 4, 0)
        decay = torch.full((H,), 0.99, device=dev)
        kw = {}
        if prompt:
            kw = dict(max_q_len=per, scratch=torch.empty(ops.decay_attn_chunked_scratch_floats(n_seqs, per, H, hd, hd), device=dev))
        st2 = torch.zeros(n_seqs, H, hd, hd, device=dev)
        us_decay = mb._time(lambda i: ops.decay_attn(q, k, v, decay, st2, step.slot_ids, step.seq_start, H, hd, hd, silu=False, **kw), 1, **it)
        like_decay = {"kernel": "decay_attn", "us": round(us_decay, 1), "frac": _frac(us_decay, rows * qd * (3 * 2 + 4) + 2 * st2.numel() * 4, 4.0 * rows * qd * hd, peaks)}
        note(f"{tag}_retention_recurrence", us_decay, rows * qd * (3 * 2 + 4) + 2 * st2.numel() * 4, 4.0 * rows * qd * hd, like=like_decay)
        o = torch.randn(rows, qd, device=dev)
        us = mb._time(lambda i: ops.head_norm_gate(o, H, hd, None, 1e-6, g, ops.GATE_SILU, bf), 1, **it)
        w2 = torch.ones(qd, device=dev)
        us_like = mb._time(lambda i: ops.rms_gate(o, w2, 1e-5, g, bf), 1, **it)
        nbytes = rows * qd * (4 + 2 + 2)
        note(f"{tag}_heads_norm_gate", us, nbytes, 0, like={"kernel": "rms_gate", "us": round(us_like, 1), "frac": _frac(us_like, nbytes, 0, peaks)})
        # ---- the gated delta rule: convolutions, unit vectors and scalars, the recurrence
        C = 3 * qd
        wc = torch.randn(TAPS, C, device=dev)
        rec = torch.zeros(n_seqs, TAPS - 1, C, device=dev)
        us = mb._time(lambda i: ops.short_conv(proj[:, :C], wc, rec, step.slot_ids, step.seq_start, step.tok_seq), 1, **it)
        note(f"{tag}_delta_short_conv", us, rows * C * 4, 0)
        conv = ops.short_conv(proj[:, :C], wc, rec, step.slot_ids, step.seq_start, step.tok_seq)
        ba = proj[:, 4 * qd:]
        a_log, dt = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
        us = mb._time(lambda i: ops.delta_prep(conv[:, : 2 * qd], ba, a_log, dt, H, H, hd, 1e-6, hd ** -0.5), 1, **it)
        note(f"{tag}_delta_unit_vectors_scalars", us, rows * 2 * qd * (2 + 4), 0)
        qn, kn, kq, beta, dec = ops.delta_prep(conv[:, : 2 * qd], ba, a_log, dt, H, H, hd, 1e-6, hd ** -0.5)
        st3 = torch.zeros(n_seqs, H, hd, hd, device=dev)
        us = mb._time(lambda i: ops.delta_rule(qn, kn, kq, conv[:, 2 * qd:], beta, dec, st3, step.slot_ids, step.seq_start, H, H, hd, hd), 1, **it)
        note(f"{tag}_delta_recurrence", us, rows * qd * (2 * 4 + 2 + 4) + 2 * st3.numel() * 4, 6.0 * rows * qd * hd, like=like_decay)
    ops.tc_status_check()
    return out


def run(sizes, T: int, batch: int, ctx: int, steps: int, warmup: int, peaks: dict, kernels: bool = True) -> dict:
    result = {"design": "Namalix", "beside": "Revirax at equal width, heads, kv heads, head size, layers and vocabulary; its window never binds, "
              "its dense feed-forward has the weights of the experts a token uses",
              "layers": LAYERS, "dtype": "bf16", "prompt_tokens": T, "decode_batch": batch, "decode_context": ctx, "peaks": peaks, "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        row = {"config": z}
        for who, cfg in (("namalix", namalix_config(z)), ("revirax", revirax_config(dict(z, chunk=4 * max(T, ctx), mem_heads=0)))):
            t = step_times(cfg, T, batch, ctx, steps, warmup)
            row[who] = {
                "prefill_ms": round(t["prefill_ms"], 3), "prefill_tokens_per_s": round(T / t["prefill_ms"] * 1e3, 1),
                "decode_ms": round(t["decode_ms"], 4), "decode_tokens_per_s": round(batch / t["decode_ms"] * 1e3, 1),
            }
        if kernels:
            row["kernels"] = kernel_table(z, T, batch, ctx, peaks)
        result["sizes"][name] = row
    return result
