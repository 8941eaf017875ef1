"""Causal grouped-query attention over the paged cache."""

from __future__ import annotations

import math
from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.device import sm_count
from ..kernels.linear import linear, linear_to_stream
from ..spec import PartSpec
from .base import MIXERS, POSITIONS, KVNeed, Mixer, ParamInfo

# one-warp blocks of the decode kernel that an SM holds at once (four at head size 128, its shared
# memory's limit): measured best when the splits fill the GPU once and no more
_DECODE_BLOCKS_PER_SM = 4
_DECODE_HEADS_PER_BLOCK = 8


# the four-warp kernel for head sizes 64 and 128: two blocks per SM; a split shorter than four pages costs
# more in the merge than it gains (measured at one sequence of 4096: 16 splits 7.5 us, 37 splits 8.8)
_QKV_PARTIALS_MAX_ROWS = 128
_DECODE_TMA_BLOCKS_PER_SM = 2
_DECODE_TMA_MIN_PAGES = 4


def decode_splits(n_seqs: int, num_heads: int, num_kv_heads: int, kv_len: int, head_dim: int = 0, sms: int = 0) -> int:
    """How many pieces to cut the key range into, from shapes only (head_dim tells which of the two
    decode kernels will run; sms: the GPU's multiprocessors, asked from the current device if 0)."""
    sms = sms or sm_count()
    group = num_heads // num_kv_heads
    per_split = n_seqs * num_kv_heads * ((group + _DECODE_HEADS_PER_BLOCK - 1) // _DECODE_HEADS_PER_BLOCK)
    tiles = max(1, (kv_len + ops.PAGE_SIZE - 1) // ops.PAGE_SIZE)
    if head_dim in ops.ATTN_DECODE_TMA_HEAD_DIMS:
        want = _DECODE_TMA_BLOCKS_PER_SM * sms // per_split
        return max(1, min(want, (tiles + _DECODE_TMA_MIN_PAGES - 1) // _DECODE_TMA_MIN_PAGES, 64))
    want = _DECODE_BLOCKS_PER_SM * sms // per_split
    return max(1, min(want, tiles, 64))


_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "gate": "g", "sink": "sink", "head_mix": "talk",
          "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias", "q_norm": "q_norm.weight",
          "k_norm": "k_norm.weight", "head_bias": "pb", "value_mix": "vmix"}


@MIXERS.register("attention")
class Attention(Mixer):
    """q = Wq xn, k = Wk xn, v = Wv xn; positions encoded into q and k; k, v stored in the
    cache; each query attends to its sequence's keys up to its own position (all of
    them, or the last `window`); the heads' results go through Wo
    (src/model.rs:1253-1301, src/backend/cpu.rs:363-433).  Query head h reads kv head
    h // (H / K); the score scale is 1/sqrt(head_dim) unless `scale` names another.

    params: hidden_size, num_heads, num_kv_heads, head_dim, window (0 = all keys),
            position (a PartSpec of the position family).
    Optional params, each absent from a plain attention: value_dim (the size of a value head where it differs
    from head_dim), scale, sink (bool: exp(sink_h) joins the softmax's denominator), head_mix (bool: the heads' scaled
    scores are mixed by a learned [H, H] matrix before the softmax), gate (bool: the concatenated heads are multiplied
    by sigmoid(Wg xn) before Wo), bias (bool: q, k, v and the output projection have biases; "qkv": only q, k, v),
    out_scale (a constant factor on the result, applied in 32-bit where the heads' result is formed), sink "zero" (a sink
    whose score is the constant 0: the softmax's denominator grows by one, no tensor), qk_norm (None, or the eps of an RMS norm
    of every q and k head over the head's numbers, with one learned weight row for the q heads and one for the k heads, after
    the biases and before the rotation), softcap (0, or the cap c of s <- c tanh(s / c) on the scaled scores), chunk (0, or the
    size of the chunks, counted from position 0, outside of which a query sees nothing; the cache gives back the pages of
    chunks that are over), weights ("softmax", or "logistic": no softmax at all; a visible key's weight is logistic(score +
    head_bias_h), nothing is normalised over the keys, and `head_mix` then mixes the heads' WEIGHTS, after the logistic function),
    head_bias (bool: one learned number per head, added to the score; with logistic weights only), gate "head" (one gate number
    per head instead of one per value: Wg is [H, d]), value_mix (None, or {"key": a name, "role": "source" or "mix"}: the
    "source" layer leaves the values it projected for the step's tokens under that name, a "mix" layer stores and attends to
    (1 - lambda) v + lambda v_source, lambda a learned number; both kinds of layer have the tensor), names (tensor names after the
    prefix, keys q k v o gate sink head_mix q_bias k_bias v_bias o_bias q_norm k_norm head_bias value_mix).
    tensors: <prefix>q_proj.weight [H hd, d], k_proj.weight [K hd, d], v_proj.weight [K vd, d],
             o_proj.weight [d, H vd]; with the options also g [H vd, d], sink [H], talk [H, H] and the biases.
             q, k, v (and the gate) are kept as one matrix so that one product
             serves them all (src/backend/cuda.rs:423-442).

    A plain attention, with or without a sink, runs on the kernels built for it (tensor-core prompt attention, TMA-fed
    decode attention, the rotation fused with the cache write or with the decode kernel).  With any other option (and with a
    sink in a 32-bit run, or at a head size that is no multiple of 8) it runs on `qkv_prep` and then, in bfloat16 at sizes in
    multiples of 8, on the tensor-core kernels of csrc/attention_mix_mma.cu (`flash_mix` for prompts, `flash_mix_decode` for
    single tokens, mixed scores through `fold_queries`), else on `attn_ext` (csrc/attention_ext.cu), which takes every option,
    every size and both element types."""

    takes_out = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.H = int(self._param("num_heads"))
        self.K = int(self._param("num_kv_heads"))
        self.hd = int(self._param("head_dim"))
        self.window = int(self._param("window"))
        self.vd = int(spec.params.get("value_dim") or self.hd)
        self.has_sink = bool(spec.params.get("sink", False))
        self.zero_sink = spec.params.get("sink") == "zero"
        qk_norm = spec.params.get("qk_norm")
        self.qk_norm_eps = None if qk_norm is None else float(qk_norm)
        self.softcap = float(spec.params.get("softcap", 0.0) or 0.0)
        self.chunk = int(spec.params.get("chunk", 0) or 0)
        if self.softcap < 0 or self.chunk < 0:
            raise ConfigError(f"attention: softcap {self.softcap} and chunk {self.chunk} must not be negative")
        self.has_mix = bool(spec.params.get("head_mix", False))
        self.has_gate = bool(spec.params.get("gate", False))
        self.head_gate = spec.params.get("gate") == "head"
        weights = spec.params.get("weights", "softmax")
        if weights not in ("softmax", "logistic"):
            raise ConfigError(f"attention: weights '{weights}' are not built (known: softmax, logistic)")
        self.logistic = weights == "logistic"
        self.has_head_bias = bool(spec.params.get("head_bias", False))
        self.value_mix = spec.params.get("value_mix")
        if self.value_mix is not None and (self.value_mix.get("role") not in ("source", "mix") or not self.value_mix.get("key")):
            raise ConfigError("attention: value_mix needs a key and the role 'source' or 'mix'")
        if (self.has_head_bias or self.head_gate) and not self.logistic:
            raise ConfigError("attention: a bias per head and a gate per head are built for logistic weights only")
        self.has_bias = bool(spec.params.get("bias", False))
        self.has_o_bias = self.has_bias and spec.params.get("bias") != "qkv"
        self.out_scale = float(spec.params.get("out_scale", 1.0))
        self.names = dict(_NAMES, **dict(spec.params.get("names", {})))
        if min(self.H, self.K, self.hd, self.vd) <= 0 or self.H % self.K:
            raise ConfigError(f"attention: {self.H} heads are not a multiple of {self.K} kv heads")
        pos_spec = self._param("position")
        if not isinstance(pos_spec, PartSpec):
            raise ConfigError("attention: 'position' must be a PartSpec")
        self.position = POSITIONS.build(pos_spec, runtime)
        magnitude = float(getattr(self.position, "magnitude", 1.0))
        # what the kernels built for a plain attention take: equal key and value sizes, at most a sink beside the plain softmax
        # (the 32-bit attention kernel has none), and in bfloat16 a head size that moves in 16-byte pieces
        plain = self.vd == self.hd and not (self.has_mix or self.has_gate or self.has_bias) and self.out_scale == 1.0 and magnitude == 1.0
        plain = plain and not (self.zero_sink or self.qk_norm_eps is not None or self.softcap or self.chunk)
        plain = plain and not (self.logistic or self.value_mix is not None)
        if self.logistic and (self.has_sink or self.zero_sink):
            raise ConfigError("attention: logistic weights have no denominator for a sink to join")
        if self.value_mix is not None and self.has_bias:
            raise ConfigError("attention: value mixing beside biases is not built")
        if plain and self.has_sink:
            plain = runtime.dtype != torch.float32 and self.hd % 8 == 0
        self.extended = not plain
        if max(self.hd, self.vd) > 256:
            raise ConfigError(f"attention: head sizes {self.hd} / {self.vd} are above 256, the most the attention kernels built here take")
        if self.extended:
            if self.has_mix and self.H > 32:
                raise ConfigError(f"attention: the scores of {self.H} heads cannot be mixed, the kernel built here takes 32")
            rotary_dim = int(getattr(self.position, "rotary_dim", 0))
            if rotary_dim and not hasattr(self.position, "inv_freq"):
                raise ConfigError("attention: with its options the mixer rotates by a frequency table itself and needs a 'rotary' position part (or none)")
            self.rotation = (getattr(self.position, "inv_freq", None), rotary_dim, bool(getattr(self.position, "interleaved", False)), magnitude)
        elif self.hd % 8 and runtime.dtype != torch.float32:
            raise ConfigError(
                f"attention: the bfloat16 kernels move a head in 16-byte pieces and need head_dim to be a multiple of 8, got {self.hd} "
                f"(a float32 run takes any head size up to 256)")
        self.scale = float(spec.params.get("scale") or 1.0 / math.sqrt(self.hd))
        self.qd, self.kvd, self.vvd, self.od = self.H * self.hd, self.K * self.hd, self.K * self.vd, self.H * self.vd
        self.gd = self.H if self.head_gate else self.od  # rows of the gate's matrix
        self.head_bias = self.v_lambda = None
        self.w_qkv = None
        self.w_o = None
        self.b_in = self.b_o = self.sink = self.mix = self.w_q_norm = self.w_k_norm = None
        self.fold_matrix = None  # what `fold_queries` mixes by in a decode step: the mixing matrix, or the identity

    def cache_need(self):
        return KVNeed(self.K, self.hd, self.window, value_dim=self.vd if self.vd != self.hd else None, chunk=self.chunk)

    def children(self):
        return (self.position,)

    def param_infos(self) -> Dict[str, ParamInfo]:
        p, n = self.prefix, self.names
        infos = {
            p + n["q"]: ParamInfo((self.qd, self.d)),
            p + n["k"]: ParamInfo((self.kvd, self.d)),
            p + n["v"]: ParamInfo((self.vvd, self.d)),
            p + n["o"]: ParamInfo((self.d, self.od)),
        }
        if self.has_gate:
            infos[p + n["gate"]] = ParamInfo((self.gd, self.d))
        if self.has_head_bias:
            infos[p + n["head_bias"]] = ParamInfo((self.H,), "scalars", centre=0.0)
        if self.value_mix is not None:
            infos[p + n["value_mix"]] = ParamInfo((), "scalars", centre=0.5)
        if self.has_sink and not self.zero_sink:
            infos[p + n["sink"]] = ParamInfo((self.H,), "scalars")
        if self.qk_norm_eps is not None:
            infos[p + n["q_norm"]] = ParamInfo((self.hd,), "scalars", centre=1.0)
            infos[p + n["k_norm"]] = ParamInfo((self.hd,), "scalars", centre=1.0)
        if self.has_mix:
            infos[p + n["head_mix"]] = ParamInfo((self.H, self.H), "scalars")
        if self.has_bias:
            for key, size in (("q_bias", self.qd), ("k_bias", self.kvd), ("v_bias", self.vvd), ("o_bias", self.d)):
                if key != "o_bias" or self.has_o_bias:
                    infos[p + n[key]] = ParamInfo((size,), "scalars", centre=0.0)
        return infos

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = self.prefix, self.names
        parts = [tensors[p + n["q"]], tensors[p + n["k"]], tensors[p + n["v"]]]
        if self.has_gate:
            parts.append(tensors[p + n["gate"]])
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()
        if self.zero_sink:
            self.sink = torch.zeros(self.H, dtype=torch.float32, device=self.w_o.device)
        elif self.has_sink:
            self.sink = tensors[p + n["sink"]].contiguous()
        if self.qk_norm_eps is not None:
            self.w_q_norm, self.w_k_norm = tensors[p + n["q_norm"]].contiguous(), tensors[p + n["k_norm"]].contiguous()
        if self.has_mix:
            self.mix = tensors[p + n["head_mix"]].contiguous()
        if self.has_head_bias:
            self.head_bias = tensors[p + n["head_bias"]].contiguous()
        if self.value_mix is not None and self.value_mix["role"] == "mix":
            self.v_lambda = tensors[p + n["value_mix"]].to(torch.float32).reshape(1).contiguous()
        if self.has_bias:
            self.b_in = torch.cat([tensors[p + n["q_bias"]], tensors[p + n["k_bias"]], tensors[p + n["v_bias"]]]).contiguous()
            if self.has_o_bias:
                self.b_o = (tensors[p + n["o_bias"]] * self.out_scale).contiguous()

    def output_bias(self):
        return self.b_o

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        a, w_o = self.forward_unprojected(xn, step, cache, shared_cache)
        return linear_to_stream(a, w_o)

    def _forward_extended(self, xn: torch.Tensor, step, cache, shared_cache: bool, out):
        if shared_cache:
            raise ConfigError("attention: a layer that reads another layer's cache cannot have this mixer's options")
        proj = linear(xn, self.w_qkv)
        inv_freq, rotary_dim, interleaved, magnitude = self.rotation
        v_src = None
        if self.value_mix is not None:
            key = self.value_mix["key"]
            if self.value_mix["role"] == "source":  # (its rows are not touched again: the values are stored in the pages as they are)
                step.shared[key] = proj[:, self.qd + self.kvd : self.qd + self.kvd + self.vvd]
            else:
                v_src = step.shared.get(key)
                if v_src is None or tuple(v_src.shape) != (proj.shape[0], self.vvd):
                    raise ConfigError(f"attention: no values '{key}' of {self.vvd} numbers a token were left by an earlier layer of this step")
        ops.qkv_prep(
            proj, self.b_in, step.tok_pos, step.tok_seq, cache.block_table, cache.k_pages, cache.v_pages, inv_freq, magnitude,
            self.H, self.K, self.hd, self.vd, rotary_dim, interleaved, q_norm=self.w_q_norm, k_norm=self.w_k_norm,
            norm_eps=self.qk_norm_eps or 0.0, v_src=v_src, v_lambda=self.v_lambda if v_src is not None else None,
        )
        gate = proj[:, self.qd + self.kvd + self.vvd :] if self.has_gate else None
        return self._attend(proj, gate, step, cache, out), self.w_o

    def _attend(self, proj: torch.Tensor, gate, step, cache, out):
        """The attention itself over rows whose queries are ready and whose keys and values are in the cache.  bfloat16 runs take
        the tcgen05 prompt kernel and the TMA-fed decode kernel where the sizes are theirs (equal key and value sizes of 64 or
        128, no mixed scores, no gate), else the tensor-core kernel for unequal sizes, mixed scores and gates; 32-bit runs and
        the remaining sizes take the general kernel."""
        bf = self.rt.dtype == torch.bfloat16
        if self.logistic:
            return self._attend_logistic(proj, gate, step, cache, out)
        if (bf and self.hd == self.vd and self.hd in ops.FLASH_TC_HEAD_DIMS and not self.has_mix and gate is None and self.out_scale == 1.0
                and proj.stride(0) % 8 == 0 and proj.data_ptr() % 16 == 0):
            direct = out is not None and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0 and out.stride(1) == 1
            if step.decode_only and self.hd in ops.ATTN_DECODE_TMA_HEAD_DIMS:
                keys = min(self.window, step.plan_kv_len) if self.window else step.plan_kv_len
                keys = min(self.chunk, keys) if self.chunk else keys
                n_splits = decode_splits(step.n_seqs, self.H, self.K, keys, self.hd)
                scratch = self.rt.workspace.get("attn_decode", ops.attn_decode_scratch_floats(step.n_seqs, self.H, self.hd, n_splits), torch.float32)
                a = ops.attn_decode(
                    proj, cache.k_pages, cache.v_pages, cache.block_table, step.seq_len, self.H, self.K, self.hd, n_splits, scratch,
                    window=self.window, scale=self.scale, sink=self.sink, chunk=self.chunk, softcap=self.softcap, impl="tma",
                    out=out if direct else None,
                )
            else:
                a = ops.flash_prefill_tc(
                    proj, cache.k_pages, cache.v_pages, cache.block_table, step.seq_start, step.seq_pos0, step.max_q_len, self.H, self.K,
                    self.hd, window=self.window, scale=self.scale, sink=self.sink, chunk=self.chunk, softcap=self.softcap,
                    out=out if direct else None,
                )
            if out is not None and a is not out:
                out.copy_(a)
                a = out
            return a
        parts = self.K if self.has_mix else 1
        if (bf and ops.flash_mix_takes(self.hd, self.vd, parts) and proj.stride(0) % 8 == 0
                and (out is None or (out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0)) and (self.qd + self.kvd + self.vvd) % 2 == 0):
            if step.decode_only and ops.flash_mix_decode_takes(self.H, self.K, self.hd, self.vd):
                # single tokens: all heads of a sequence are the rows of one block, which reads a key tile once for all of them;
                # the key range is cut into parts of a page or more so that the blocks fill the GPU (a block is one or two warps: short chains matter more than few parts)
                if self.fold_matrix is None:
                    self.fold_matrix = self.mix if self.has_mix else torch.eye(self.H, dtype=torch.float32, device=proj.device)
                qf = ops.fold_queries(proj, self.fold_matrix, self.H, self.K, self.hd)
                keys = min(self.window, step.plan_kv_len) if self.window else step.plan_kv_len
                keys = min(self.chunk, keys) if self.chunk else keys
                pages = (keys + ops.PAGE_SIZE - 1) // ops.PAGE_SIZE + 1
                n_splits = max(1, min(2 * sm_count(proj.device) // step.n_seqs, pages, 64))
                scratch = self.rt.workspace.get("flash_mix_decode", ops.flash_mix_decode_scratch_floats(step.n_seqs, self.H, self.vd, n_splits), torch.float32)
                return ops.flash_mix_decode(
                    qf, cache.k_pages, cache.v_pages, cache.block_table, step.seq_pos0, self.H, self.K, self.hd, self.vd, self.scale,
                    n_splits, scratch, window=self.window, sink=self.sink, gate=gate, out_scale=self.out_scale, out=out, chunk=self.chunk,
                    softcap=self.softcap,
                )
            # the tensor-core kernel for prompts (and single tokens of sizes the decode kernel does not take); mixed scores come
            # from folded queries
            q = ops.fold_queries(proj, self.mix, self.H, self.K, self.hd) if self.has_mix else proj
            return ops.flash_mix(
                q, cache.k_pages, cache.v_pages, cache.block_table, step.seq_start, step.seq_pos0, step.max_q_len, self.H, self.K,
                self.hd, self.vd, self.scale, window=self.window, sink=self.sink, folded=self.has_mix, gate=gate, out_scale=self.out_scale,
                out=out, chunk=self.chunk, softcap=self.softcap,
            )
        return ops.attn_ext(
            proj, cache.k_pages, cache.v_pages, cache.block_table, step.tok_seq, step.tok_pos, self.H, self.K, self.hd, self.vd,
            self.scale, window=self.window, sink=self.sink, mix=self.mix, gate=gate, out_scale=self.out_scale, out=out, chunk=self.chunk,
            softcap=self.softcap,
        )

    def _attend_logistic(self, proj: torch.Tensor, gate, step, cache, out):
        """Attention with logistic weights (csrc/attention_sigmoid.cu): bfloat16 runs at key and value sizes in multiples of 8 up to
        128 on the tensor cores (a decode step's key range cut into runs of pages so that the blocks fill the GPU), everything
        else on the general kernel, whose sums have one fixed order."""
        if (self.rt.dtype == torch.bfloat16 and ops.sigmoid_attn_mma_takes(self.hd, self.vd, self.H) and proj.stride(0) % 8 == 0
                and proj.data_ptr() % 16 == 0):
            T, mixed = proj.shape[0], self.mix is not None
            parts = 1
            if step.decode_only:
                keys = min(self.window, step.plan_kv_len) if self.window else step.plan_kv_len
                keys = min(self.chunk, keys) if self.chunk else keys
                pages = (keys + ops.PAGE_SIZE - 1) // ops.PAGE_SIZE + (1 if (self.window or self.chunk) else 0)
                blocks = step.n_seqs * self.K * (self.K if mixed else 1)  # a block's rows are the heads of one kv head
                parts = max(1, min(4 * sm_count(proj.device) // max(blocks, 1), pages, 64))
            scratch = self.rt.workspace.get("sigmoid_attn_parts", ops.sigmoid_attn_mma_scratch_floats(T, self.H, self.K, self.vd, mixed, parts), torch.float32)
            return ops.sigmoid_attn_mma(
                proj, cache.k_pages, cache.v_pages, cache.block_table, step.seq_start, step.seq_pos0, step.max_q_len, self.H, self.K, self.hd,
                self.vd, self.scale, scratch, parts=parts, head_bias=self.head_bias, mix=self.mix, gate=gate, softcap=self.softcap,
                window=self.window, chunk=self.chunk, out_scale=self.out_scale, out=out,
            )
        return ops.sigmoid_attn(
            proj, cache.k_pages, cache.v_pages, cache.block_table, step.tok_seq, step.tok_pos, self.H, self.K, self.hd, self.vd, self.scale,
            head_bias=self.head_bias, mix=self.mix, gate=gate, softcap=self.softcap, window=self.window, chunk=self.chunk,
            out_scale=self.out_scale, out=out,
        )

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False, out=None):
        """out: None, or a [T, H value_dim] view (dense rows, any row stride) that receives the heads' result."""
        if self.extended:
            return self._forward_extended(xn, step, cache, shared_cache, out)
        a, w_o = self._forward_plain(xn, step, cache, shared_cache)
        if out is not None:
            out.copy_(a)
            a = out
        return a, w_o

    def _forward_plain(self, xn: torch.Tensor, step, cache, shared_cache: bool = False):
        # a decode step of a bfloat16 run at head size 64 or 128: the attention kernel turns the queries and the
        # new key and stores key and value itself, if the position encoding is one it knows how to apply
        fusion = None
        if step.decode_only and self.rt.dtype == torch.bfloat16 and self.hd in ops.ATTN_DECODE_TMA_HEAD_DIMS:
            fusion = self.position.decode_fusion()
        # the keys and values may be another run's: then only the queries are projected.  The fused attention
        # kernel also takes the projection as partial sums over slices of k, which lets a product with few
        # output tiles use all SMs (measured at the 8B sizes: 3 % of the step gained at 16, 24 and 64 sequences)
        w = self.w_qkv[: self.qd] if shared_cache else self.w_qkv
        qkv = linear_to_stream(xn, w) if (fusion is not None and xn.shape[0] <= _QKV_PARTIALS_MAX_ROWS) else linear(xn, w)
        if fusion is None:
            self.position.write_qk(qkv, step, cache, self.H, self.K, self.hd, write_kv=not shared_cache)
        if self.rt.dtype == torch.float32:
            a = ops.attn_generic(
                qkv, cache.k_pages, cache.v_pages, cache.block_table, step.tok_seq, step.tok_pos,
                self.H, self.K, self.hd, window=self.window, scale=self.scale,
            )
        elif step.decode_only:
            n_splits = decode_splits(step.n_seqs, self.H, self.K, step.plan_kv_len, self.hd)
            scratch = self.rt.workspace.get(
                "attn_decode", ops.attn_decode_scratch_floats(step.n_seqs, self.H, self.hd, n_splits), torch.float32
            )
            # With one split per sequence the attention kernel writes the result itself.  With more, a
            # second kernel adds the splits up: letting the block that finishes last do that (the kernel
            # can) measured slower at batch 1 and 8 (its serial tail costs more than the small kernel).
            counters = None
            if self.hd in ops.ATTN_DECODE_TMA_HEAD_DIMS and n_splits == 1:
                groups = self.K * ((self.H // self.K + _DECODE_HEADS_PER_BLOCK - 1) // _DECODE_HEADS_PER_BLOCK)
                counters = self.rt.workspace.get("attn_decode_counters", step.n_seqs * groups, torch.int32, zeroed=True)
            a = ops.attn_decode(
                qkv, cache.k_pages, cache.v_pages, cache.block_table, step.seq_len, self.H, self.K, self.hd,
                n_splits, scratch, window=self.window, scale=self.scale, counters=counters, sink=self.sink,
                **({} if fusion is None else dict(
                    fuse=1 if shared_cache else 2, inv_freq=fusion[0], rotary_dim=fusion[1], interleaved=fusion[2])),
            )
        elif self.hd in ops.FLASH_TC_HEAD_DIMS:
            a = ops.flash_prefill_tc(
                qkv, cache.k_pages, cache.v_pages, cache.block_table, step.seq_start, step.seq_pos0,
                step.max_q_len, self.H, self.K, self.hd, window=self.window, scale=self.scale, sink=self.sink,
            )
        else:
            a = ops.flash_prefill(
                qkv, cache.k_pages, cache.v_pages, cache.block_table, step.seq_start, step.seq_pos0,
                step.max_q_len, self.H, self.K, self.hd, window=self.window, scale=self.scale, sink=self.sink,
            )
        return a, self.w_o


def chunked_attention_runner(proj, k_pages, v_pages, block_table, step, num_heads: int, num_kv_heads: int, kdim: int, vdim: int, scale: float,
                             chunk: int, softcap: float, sink, window: int = 0, workspace=None):
    """A callable that runs the attention of `Attention` (the kernel choice included) over ready rows, for timing it alone.
    step: tok_seq, tok_pos, seq_start, seq_pos0, seq_len (or none: positions after the step), max_q_len, n_seqs, decode_only."""
    from types import SimpleNamespace

    class _Scratch:
        def __init__(self):
            self.held = {}

        def get(self, name, numel, dtype, zeroed=False):
            buf = self.held.get(name)
            if buf is None or buf.numel() < numel or buf.dtype != dtype:
                buf = self.held[name] = torch.zeros(int(numel), dtype=dtype, device=proj.device)
            return buf

    if not hasattr(step, "seq_len"):
        step.seq_len = (step.seq_pos0 + (step.seq_start[1:] - step.seq_start[:-1])).to(torch.int32)
    if not hasattr(step, "plan_kv_len"):
        step.plan_kv_len = int(step.seq_len.max())
    part = SimpleNamespace(
        rt=SimpleNamespace(dtype=proj.dtype, workspace=workspace or _Scratch()), H=num_heads, K=num_kv_heads, hd=kdim, vd=vdim, scale=scale,
        window=window, chunk=chunk, softcap=softcap, sink=sink, mix=None, has_mix=False, out_scale=1.0, fold_matrix=None, logistic=False,
        qd=num_heads * kdim, kvd=num_kv_heads * kdim, vvd=num_kv_heads * vdim,
    )
    cache = SimpleNamespace(k_pages=k_pages, v_pages=v_pages, block_table=block_table)
    return lambda: Attention._attend(part, proj, None, step, cache, None)


def logistic_attention_runner(proj, gate, k_pages, v_pages, block_table, step, num_heads: int, num_kv_heads: int, kdim: int, vdim: int, scale: float,
                              softcap: float, head_bias, mix, window: int = 0, chunk: int = 0, workspace=None):
    """A callable that runs the attention with logistic weights as `Attention` does (the kernel choice included) over ready rows,
    for testing and timing it alone.  gate: [T, >= H] rows or None.  step: tok_seq, tok_pos, seq_start, seq_pos0, max_q_len, n_seqs,
    decode_only, plan_kv_len."""
    from types import SimpleNamespace

    class _Scratch:
        def __init__(self):
            self.held = {}

        def get(self, name, numel, dtype, zeroed=False):
            buf = self.held.get(name)
            if buf is None or buf.numel() < numel or buf.dtype != dtype:
                buf = self.held[name] = torch.zeros(int(numel), dtype=dtype, device=proj.device)
            return buf

    part = SimpleNamespace(
        rt=SimpleNamespace(dtype=proj.dtype, workspace=workspace or _Scratch()), H=num_heads, K=num_kv_heads, hd=kdim, vd=vdim, scale=scale,
        window=window, chunk=chunk, softcap=softcap, head_bias=head_bias, mix=mix, out_scale=1.0,
    )
    cache = SimpleNamespace(k_pages=k_pages, v_pages=v_pages, block_table=block_table)
    return lambda: Attention._attend_logistic(part, proj, gate, step, cache, None)
