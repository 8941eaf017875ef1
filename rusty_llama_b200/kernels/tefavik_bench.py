"""Tefavik beside Revirax (the library's closest model: a linear attention with a state per head, and a parallel layer of a
masked softmax attention and a recurrent unit) at equal sizes: prompt-step and decode-step throughput through the engine, and
every kernel that only Tefavik uses timed alone beside the kernel of Revirax or Llama that does the like work.

    python bench.py --design tefavik [--design-sizes small,lite,wide]

Sizes resemble real models' layers (random weights, four layers: gla, parallel, gla, parallel; the whole vocabulary).  Revirax
beside it has the same width, heads, kv heads, head size, layer count and vocabulary; its window is Tefavik's chunk, and its
dense feed-forward has as many weights as the experts that a token of Tefavik uses.  Every kernel's fraction is what it must
move (bytes, against the measured copy rate) or compute (flops, against the measured bfloat16 matrix rate), whichever bound
is the tighter one, divided by the time it took.
"""

from __future__ import annotations

import math
from types import SimpleNamespace
from typing import Dict

import torch

from . import microbench as mb
from . import ops
from .design_bench import _frac, step_times

SIZES = {
    "small": dict(width=1024, heads=8, kv_heads=2, hd=128, chunk=512, mem_heads=4, experts=8, top=2, eff=1408, vocab=32000),
    "lite": dict(width=2048, heads=16, kv_heads=4, hd=128, chunk=1024, mem_heads=8, experts=16, top=2, eff=2816, vocab=32000),
    "wide": dict(width=4096, heads=32, kv_heads=8, hd=128, chunk=1024, mem_heads=16, experts=16, top=2, eff=4096, vocab=32000),
}
LAYERS = 4
DECAY_RANK = 16


def tefavik_config(z: dict) -> dict:
    H, G, hd = z["heads"], z["kv_heads"], z["hd"]
    left = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": 1.0 / math.sqrt(hd), "softcap": 30.0, "mask": {"size": z["chunk"]},
            "rot": {"base": 10000.0, "dims": hd}}
    right = {"heads": z["mem_heads"], "dim": hd, "vdim": hd, "gate_cap": 15.0}
    gla = {"heads": H, "dim": hd, "vdim": hd, "tau": 8.0}
    mlp = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["eff"], "limit": 7.0}}
    kinds = [("gla", gla), ("parallel", {"left": left, "right": right})]
    layers = [{"type": t, "mixer": m, "mlp": mlp} for t, m in (kinds[i % 2] for i in range(LAYERS))]
    return {"architecture": "Tefavik", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "layers": layers, "loop": None}


def revirax_config(z: dict) -> dict:
    H, G, hd = z["heads"], z["kv_heads"], z["hd"]
    left = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": 1.0 / math.sqrt(hd), "mask": {"size": z["chunk"]},
            "rot": {"base": 10000.0, "dims": hd // 2, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    lightning = {"heads": H, "dim": hd, "vdim": hd, "decay": [1.0 - 2.0 ** (-3 - 5 * i / max(H - 1, 1)) for i in range(H)]}
    parallel = {"left": left, "right": {"width": z["width"]}, "left_scale": 0.7, "right_scale": 0.7}
    mlp = {"kind": "dense", "ff": z["top"] * z["eff"] * 3 // 2}
    kinds = [("lightning", lightning), ("parallel", parallel)]
    layers = [{"type": t, "mixer": m, "mlp": mlp} for t, m in (kinds[i % 2] for i in range(LAYERS))]
    return {"architecture": "Revirax", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "layers": layers}


def kernel_table(z: dict, T: int, batch: int, ctx: int, peaks: dict) -> Dict[str, dict]:
    """Each kernel of the design alone, at a prompt step of T tokens (one sequence) and a decode step of `batch` sequences at `ctx`."""
    from ..parts import attention as attention_part
    from ..parts import gated_recurrent as recurrent_part

    dev, bf = "cuda:0", torch.bfloat16
    H, G, hd, C, MH = z["heads"], z["kv_heads"], z["hd"], z["chunk"], z["mem_heads"]
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
        )
        # ---- the chunked, capped attention with its zero sink: norms of q and k, rotation and cache write; then the attention
        pages = (pos0 + per + 63) // 64
        kp = torch.randn(n_seqs * pages, G, 64, hd, device=dev, dtype=bf)
        vp = torch.randn(n_seqs * pages, G, 64, hd, device=dev, dtype=bf)
        table = torch.randperm(n_seqs * pages, device=dev).to(torch.int32).view(n_seqs, pages).contiguous()
        qkv = torch.randn(rows, (H + 2 * G) * hd, device=dev, dtype=bf)
        bias = torch.zeros((H + 2 * G) * hd, device=dev)
        freq = torch.rand(hd // 2, device=dev)
        wn = torch.ones(hd, device=dev)
        us = mb._time(lambda i: ops.qkv_prep(qkv, bias, step.tok_pos, step.tok_seq, table, kp, vp, freq, 1.0, H, G, hd, hd, hd, True,
                                             q_norm=wn, k_norm=wn, norm_eps=1e-6), 1, **it)
        us_like = mb._time(lambda i: ops.rope_kv_write(qkv, step.tok_pos, step.tok_seq, table, kp, vp, freq, H, G, hd, hd, True), 1, **it)
        nbytes = rows * ((H + G) * hd * 4 + G * hd * 4)
        note(f"{tag}_bias_norm_rotate_store", us, nbytes, 0, like={"kernel": "rope_kv_write", "us": round(us_like, 1), "frac": _frac(us_like, nbytes, 0, peaks)})
        sink = torch.zeros(H, device=dev)
        run = attention_part.chunked_attention_runner(qkv, kp, vp, table, step, H, G, hd, hd, scale, C, 30.0, sink)
        us = mb._time(lambda i: run(), 1, **it)
        keys = sum(p % C + 1 for p in range(pos0, pos0 + per)) * n_seqs
        seen = min(C, pos0 + per) if prompt else (pos0 % C + 1)
        note(f"{tag}_attention_chunked_capped_sink", us, n_seqs * seen * G * 2 * hd * 2 + rows * H * hd * 4, 4.0 * keys * H * hd,
             like=like_prefill if prompt else like_decode)
        # ---- the two recurrences: gates, the state's walk, the heads' norm and gate
        for name, heads, ext in (("gla", H, False), ("mlstm", MH, True)):
            qd = heads * hd
            proj = torch.randn(rows, 4 * qd + 2 * heads, device=dev, dtype=bf)
            q, k, v, g = (proj[:, i * qd: (i + 1) * qd] for i in range(4))
            vcols = hd + (1 if ext else 0)
            state = torch.zeros(n_seqs, heads, hd, vcols, device=dev)
            if ext:
                m_state = torch.zeros(n_seqs, heads, device=dev)
                bz = torch.zeros(heads, device=dev)
                gi, gf = proj[:, 4 * qd: 4 * qd + heads], proj[:, 4 * qd + heads:]
                us = mb._time(lambda i: ops.mlstm_gates(gi, gf, bz, bz, 15.0, m_state, step.slot_ids, step.seq_start, scan=prompt), 1, **it)
                note(f"{tag}_mlstm_gates", us, rows * heads * (4 + 12), 0)
                log_a, b, m = ops.mlstm_gates(gi, gf, bz, bz, 15.0, m_state, step.slot_ids, step.seq_start)
            else:
                zz = torch.randn(rows, qd, device=dev, dtype=bf)
                bz = torch.zeros(qd, device=dev)
                us = mb._time(lambda i: ops.gla_log_decay(zz, bz, 8.0), 1, **it)
                note(f"{tag}_gla_log_decay", us, rows * qd * 6, 0)
                log_a, b, m = ops.gla_log_decay(zz, bz, 8.0), None, None
            mixer = SimpleNamespace(H=heads, dim=hd, vdim=hd, q_scale=hd ** -0.5, rt=SimpleNamespace(workspace=_Workspace(dev)))
            us = mb._time(lambda i: recurrent_part._recurrence(mixer, q, k, v, log_a, b, state, step, ext), 1, **it)
            like = None
            if name == "gla":  # Revirax's linear attention with a constant decay per head, same sizes
                decay = torch.full((heads,), 0.99, device=dev)
                kw = {}
                if prompt:
                    kw = dict(max_q_len=per, scratch=torch.empty(ops.decay_attn_chunked_scratch_floats(n_seqs, per, heads, hd, hd), device=dev))
                st2 = torch.zeros(n_seqs, heads, hd, hd, device=dev)
                us_like = mb._time(lambda i: ops.decay_attn(q, k, v, decay, st2, step.slot_ids, step.seq_start, heads, hd, hd, silu=True, **kw), 1, **it)
                like = {"kernel": "decay_attn", "us": round(us_like, 1),
                        "frac": _frac(us_like, rows * qd * (3 * 2 + 4) + 2 * st2.numel() * 4, 4.0 * rows * qd * hd, peaks)}
            note(f"{tag}_{name}_recurrence", us, rows * qd * (3 * 2 + 4 + (4 if not ext else 0)) + 2 * state.numel() * 4, 4.0 * rows * qd * vcols, like=like)
            o = torch.randn(rows, heads * vcols, device=dev)
            w = torch.ones(heads * hd if ext else hd, device=dev)
            us = mb._time(lambda i: ops.head_norm_gate(o, heads, hd, w, 1e-6, g, ops.GATE_SIGMOID if ext else ops.GATE_SILU, bf, m=m, den_eps=1e-6), 1, **it)
            o2 = torch.randn(rows, qd, device=dev)
            w2 = torch.ones(qd, device=dev)
            us_like = mb._time(lambda i: ops.rms_gate(o2, w2, 1e-5, g, bf), 1, **it)
            nbytes = rows * qd * (4 + 2 + 2)
            note(f"{tag}_{name}_heads_norm_gate", us, nbytes, 0, like={"kernel": "rms_gate", "us": round(us_like, 1), "frac": _frac(us_like, nbytes, 0, peaks)})
    ops.tc_status_check()
    return out


class _Workspace:
    """What a part's runtime offers for scratch: one buffer per name that only grows."""

    def __init__(self, device):
        self.device, self.buffers = device, {}

    def get(self, name, numel, dtype):
        buf = self.buffers.get(name)
        if buf is None or buf.numel() < numel or buf.dtype != dtype:
            buf = self.buffers[name] = torch.empty(int(numel), dtype=dtype, device=self.device)
        return buf


def run(sizes, T: int, batch: int, ctx: int, steps: int, warmup: int, peaks: dict, kernels: bool = True) -> dict:
    result = {"design": "Tefavik", "beside": "Revirax at equal width, heads, kv heads, head size, layers and vocabulary; its window is the chunk, "
              "its dense feed-forward has the weights of the experts a token uses",
              "layers": LAYERS, "dtype": "bf16", "prompt_tokens": T, "decode_batch": batch, "decode_context": ctx, "peaks": peaks, "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        row = {"config": z}
        for who, cfg in (("tefavik", tefavik_config(z)), ("revirax", revirax_config(z))):
            t = step_times(cfg, T, batch, ctx, steps, warmup)
            row[who] = {
                "prefill_ms": round(t["prefill_ms"], 3), "prefill_tokens_per_s": round(T / t["prefill_ms"] * 1e3, 1),
                "decode_ms": round(t["decode_ms"], 4), "decode_tokens_per_s": round(batch / t["decode_ms"] * 1e3, 1),
            }
        if kernels:
            row["kernels"] = kernel_table(z, T, batch, ctx, peaks)
        result["sizes"][name] = row
    return result
