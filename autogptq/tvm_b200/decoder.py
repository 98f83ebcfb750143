"""Decoder harness around the QuantLinear path: Llama- and OPT-architecture models whose
linears are synthetic GPTQ layers, with tensor parallelism over ``torch.distributed``.

This is the step either side of the linears that the reference leaves to ``transformers``
(its benchmark drives ``model.generate``: ``end2end/autogptq-generation-inference-benchmark.py:26-49``,
``quantization/opt.py:306-354``).  Here it is a small explicit model so that one decode step can
be captured in a CUDA graph and the linears can be sharded:

* column-parallel (no exchange): fused q/k/v and fused gate/up (OPT: fc1) -- each rank owns a slice
  of the output features, i.e. whole attention heads and a slice of the FFN width;
* row-parallel (one all-reduce): o_proj and down_proj (OPT: out_proj, fc2) -- each rank owns the
  matching slice of the input features, cut on quantisation-group boundaries;
* the vocabulary projection stays dense fp16 (``modeling/_base.py:534`` keeps lm_head out of the
  quantised set) and is sharded over the vocabulary; ranks exchange their best (logit, token).

Weights are random (no checkpoints offline) but the model is ONE model at every tensor-parallel degree:
every rank draws each full layer from a seed that does not depend on the rank, cuts its shard out of it
with the rules of :mod:`tp` and drops the rest, so a run on N GPUs computes the same function as a run on
one (up to the summation order of the row-parallel layers).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _lib, ops, synth, tp
from .qlinear import QuantLinear


@dataclass
class DecoderConfig:
    arch: str = "llama"            # "llama" (RMSNorm, RoPE, SwiGLU) or "opt" (LayerNorm, learned positions, ReLU)
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    inter: int = 11008
    vocab: int = 32000
    bits: int = 4
    group_size: int = 128
    desc_act: bool = False
    max_seq: int = 768
    rope_theta: float = 10000.0
    # Random weights with the benchmark's scale distribution amplify activations ~8x per linear and
    # overflow fp16 within one decoder layer; the harness shrinks the scales so that values stay finite
    # (kernel time does not depend on the values).
    scale_mult: float = 1.0 / 16.0

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


LLAMA_7B = DecoderConfig()
OPT_66B = DecoderConfig(arch="opt", layers=64, hidden=9216, heads=72, inter=36864, vocab=50272, bits=3,
                        group_size=128, desc_act=True, max_seq=256)


def check_positions(pos: int, steps: int, max_seq: int) -> None:
    """Refuse a run that would step past the KV caches: the kernels take the position from device memory (so that a
    captured graph can advance it), which leaves this host-side check as the place where a bad request is reported."""
    if pos < 0 or steps < 0 or pos + steps > max_seq:
        raise ValueError(f"{steps} steps from position {pos} do not fit the KV caches (max_seq = {max_seq})")


def _full_layer(cfg: DecoderConfig, K: int, N: int, bias: bool, seed: int, device) -> synth.PackedLayer:
    return synth.make_layer(cfg.bits, K, N, cfg.group_size, cfg.desc_act, bias=bias, seed=seed, device=device,
                            scale_mult=cfg.scale_mult)


def _to_module(layer: synth.PackedLayer, device) -> QuantLinear:
    """A QuantLinear that owns the tensors of ``layer`` (a full layer or a shard), ready to run."""
    m = QuantLinear(layer.bits, layer.group_size, layer.K, layer.N, layer.bias is not None)
    m.qweight, m.qzeros, m.scales, m.g_idx = layer.qweight, layer.qzeros, layer.scales, layer.g_idx
    if layer.bias is not None:
        m.bias = layer.bias
    m = m.to(device)
    m.post_init()
    if m._x_perm is not None and m._g_idx_run is None:
        # rows re-ordered by group and back to k // group_size: keep only the re-ordered copy of the weights
        m.qweight = m._qweight_run
        m.g_idx = (torch.arange(layer.K, device=device) // m.groupsize).to(torch.int32)
        m._ready_for = (m.qweight.data_ptr(), m.g_idx.data_ptr())
    return m


class DecoderLayer:
    def __init__(self, cfg: DecoderConfig, idx: int, rank: int, world: int, device):
        self.cfg = cfg
        hd = cfg.head_dim
        head_sizes = [h * hd for h in tp.split_sizes(cfg.heads, world, 1)]       # columns of q (= k = v) per rank
        inter_sizes = tp.split_sizes(cfg.inter, world, cfg.group_size)          # FFN width per rank, whole groups
        self.heads_local, self.inter_local = head_sizes[rank] // hd, inter_sizes[rank]
        bias = cfg.arch == "opt"
        up_parts = 2 if cfg.arch == "llama" else 1
        seed = 10 * idx          # the same on every rank: the full layer is drawn, the shard cut out, the rest dropped
        full = _full_layer(cfg, cfg.hidden, 3 * cfg.hidden, bias, seed + 1, device)
        self.qkv = _to_module(tp.shard_column(full, rank, world, parts=3, sizes=head_sizes), device)
        full = _full_layer(cfg, cfg.hidden, cfg.hidden, bias, seed + 2, device)
        self.o = _to_module(tp.shard_row(full, rank, world, sizes=head_sizes)[0], device)
        self.o.tp_bias = full.bias          # the fused all-reduce adds the whole bias on every rank
        full_up = _full_layer(cfg, cfg.hidden, up_parts * cfg.inter, bias, seed + 3, device)
        full = _full_layer(cfg, cfg.inter, cfg.hidden, bias, seed + 4, device)
        if cfg.desc_act:
            # The FFN's second linear reads an element-wise function of the first one's output: its act-order row
            # permutation is folded into the first one's column order once, here, after which it is an ordinary
            # layer (no gather of its input, whole groups per rank).  The pair computes the same function.
            qs, perm, _ = ops.sort_rows(full.qweight.contiguous(), full.g_idx.contiguous(), cfg.bits)
            full, full_up = tp.fold_act_order(full, full_up, qs, perm, parts=up_parts)
        self.up = _to_module(tp.shard_column(full_up, rank, world, parts=up_parts, sizes=inter_sizes), device)
        self.down = _to_module(tp.shard_row(full, rank, world, sizes=inter_sizes)[0], device)
        self.down.tp_bias = full.bias
        del full, full_up
        g = torch.Generator(device=device).manual_seed(seed + 5)
        self.norm1_w = 1.0 + 0.01 * torch.randn(cfg.hidden, generator=g, device=device, dtype=torch.float16)
        self.norm2_w = 1.0 + 0.01 * torch.randn(cfg.hidden, generator=g, device=device, dtype=torch.float16)
        self.norm1_b = self.norm2_b = None
        if cfg.arch == "opt":
            self.norm1_b = torch.zeros(cfg.hidden, device=device, dtype=torch.float16)
            self.norm2_b = torch.zeros(cfg.hidden, device=device, dtype=torch.float16)
        self.k_cache: Optional[torch.Tensor] = None
        self.v_cache: Optional[torch.Tensor] = None

    def linear_bytes(self) -> int:
        tot = 0
        for m in (self.qkv, self.o, self.up, self.down):
            tot += m.qweight.numel() * 4 + m.qzeros.numel() * 4 + m.scales.numel() * 2
        return tot


def _rmsnorm(x, w, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class GPTQDecoder:
    """Batch of sequences, one token per step after the prompt; greedy sampling."""

    def __init__(self, cfg: DecoderConfig, batch: int = 1, device="cuda", group=None, fused: bool = True,
                 single: bool = False, fused_allreduce: bool = False, fold_activation: Optional[bool] = None):
        """``single=True`` builds the whole model on this device even inside a process group (the unsharded
        yardstick of a tensor-parallel run).  ``fold_activation``: decode steps of up to 8 sequences let the second
        FFN linear apply SiLU(gate) * up / ReLU as it reads its input instead of launching the element-wise kernel
        (bit-identical).  Measured for Llama-7B: slower on one GPU (367 against 383-390 tok/s: every CTA then computes
        the activation of its K slice between the dependency wait and its first product), faster from two GPUs on,
        where the slices are short and a launch is a larger share of the step (536 against 508 tok/s at TP 2).
        ``None`` picks accordingly."""
        self.cfg, self.batch = cfg, batch
        self._fold_request = fold_activation
        self.fused = fused and cfg.head_dim in (64, 128)   # decode steps use the fused helper kernels
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized() and not single) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.fold_activation = (self.world > 1) if self._fold_request is None else bool(self._fold_request)
        self.last_logits: Optional[torch.Tensor] = None   # this rank's slice of the latest logits [B, vocab_local]
        # fused_allreduce: the row-parallel linears and the token pick exchange through peer memory inside the
        # library's kernels instead of calling the process group (up to 8 rows; more rows still use it)
        self.exchange = None
        if fused_allreduce and self.world > 1:
            from .exchange import PeerExchange
            self.exchange = PeerExchange(self.device, group)
        dev = self.device
        self.layers = [DecoderLayer(cfg, i, self.rank, self.world, dev) for i in range(cfg.layers)]
        for L in self.layers:
            L.o.exchange = L.down.exchange = self.exchange
            # in a decode step small kernels sit between the GEMVs: fewer, longer K slices and a footprint of a third
            # of an SM measured fastest there (392 against 350 tokens/s on the Llama-7B architecture, one GPU)
            for mod in (L.qkv, L.o, L.up, L.down):
                mod.gemv_tuning = (2, 3)
        g = torch.Generator(device=dev).manual_seed(7)   # replicated tensors: the same seed on every rank
        self.embed = (0.02 * torch.randn(cfg.vocab, cfg.hidden, generator=g, device=dev)).half()
        self.pos_embed = None
        if cfg.arch == "opt":
            self.pos_embed = (0.02 * torch.randn(cfg.max_seq + 2, cfg.hidden, generator=g, device=dev)).half()
        self.final_norm_w = torch.ones(cfg.hidden, device=dev, dtype=torch.float16)
        self.final_norm_b = torch.zeros(cfg.hidden, device=dev, dtype=torch.float16) if cfg.arch == "opt" else None
        vocab_pad = (cfg.vocab + self.world * 8 - 1) // (self.world * 8) * (self.world * 8)
        self.vocab_local = vocab_pad // self.world
        # The vocabulary projection is drawn row by row of its transpose, so that a rank's slice holds the same
        # numbers whatever the padding (which depends on the number of ranks).
        gl = torch.Generator(device=dev).manual_seed(9000)
        head_t = (0.02 * torch.randn(cfg.vocab, cfg.hidden, generator=gl, device=dev)).half()
        lo = self.rank * self.vocab_local
        sl = head_t[lo:lo + self.vocab_local]
        if sl.shape[0] < self.vocab_local:   # the last rank's padding columns
            sl = torch.cat([sl, torch.zeros(self.vocab_local - sl.shape[0], cfg.hidden, device=dev, dtype=torch.float16)])
        self.lm_head = sl.contiguous()          # [vocab_local, hidden]: rows of the projection, streamed once per step
        del head_t
        hd = cfg.head_dim
        for L in self.layers:
            L.k_cache = torch.zeros(batch, L.heads_local, cfg.max_seq, hd, device=dev, dtype=torch.float16)
            L.v_cache = torch.zeros_like(L.k_cache)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, hd, 2, device=dev).float() / hd))
        ang = torch.arange(cfg.max_seq, device=dev).float()[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().half(), ang.sin().half()
        # device-side step state, so that a decode step can be replayed from a CUDA graph
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.tokens = torch.zeros(batch, dtype=torch.long, device=dev)
        self.positions = torch.arange(cfg.max_seq, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._pos_host = 0   # host copy of the position, for range checks

    # ---- pieces ----
    def _norm(self, x, w, b):
        if self.cfg.arch == "llama":
            return _rmsnorm(x, w)
        return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), 1e-5).to(x.dtype)

    def _all_reduce(self, t):
        if self.world > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def _row(self, mod: QuantLinear, x, input_act: int = 0):
        """A row-parallel linear: this rank's slice of the input in, the sum over ranks out.  ``input_act``: the
        activation in front of it, folded into the layer's read of ``x`` (the caller has checked ``mod.can_fold``)."""
        if self.world == 1:
            return mod.forward_act(x, input_act) if input_act else mod(x)
        if self.exchange is not None:
            return mod.forward_reduce(x, input_act)
        y = mod.forward_act(x, input_act) if input_act else mod(x)
        return self._all_reduce(y)               # the shard of rank 0 carries the bias

    def _rope(self, t, cos, sin):
        # t: [B, H, S, hd]; cos/sin: [S, hd/2]
        t1, t2 = t[..., 0::2], t[..., 1::2]
        o = torch.empty_like(t)
        o[..., 0::2] = t1 * cos - t2 * sin
        o[..., 1::2] = t1 * sin + t2 * cos
        return o

    def _layer(self, L: DecoderLayer, x, pos_idx, S: int, decode: bool):
        cfg = self.cfg
        B, hd = self.batch, cfg.head_dim
        h = self._norm(x, L.norm1_w, L.norm1_b)
        qkv = L.qkv(h.reshape(B * S, cfg.hidden)).reshape(B, S, 3, L.heads_local, hd)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))           # [B, H, S, hd]
        if cfg.arch == "llama":
            cos, sin = self.cos.index_select(0, pos_idx), self.sin.index_select(0, pos_idx)
            q, k = self._rope(q, cos, sin), self._rope(k, cos, sin)
        L.k_cache.index_copy_(2, pos_idx, k)
        L.v_cache.index_copy_(2, pos_idx, v)
        if decode:
            mask = (self.positions <= self.pos)[None, None, None, :]          # attend to the cache up to this step
            att = F.scaled_dot_product_attention(q, L.k_cache, L.v_cache, attn_mask=mask)
        else:
            att = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        att = att.transpose(1, 2).reshape(B * S, L.heads_local * hd)
        x = x + self._row(L.o, att).reshape(B, S, cfg.hidden)
        h = self._norm(x, L.norm2_w, L.norm2_b)
        u = L.up(h.reshape(B * S, cfg.hidden))
        if cfg.arch == "llama":
            act = F.silu(u[:, :L.inter_local]) * u[:, L.inter_local:]
        else:
            act = F.relu(u)
        x = x + self._row(L.down, act.contiguous()).reshape(B, S, cfg.hidden)
        return x

    def _embed(self, tokens, pos_idx):
        x = self.embed.index_select(0, tokens.reshape(-1)).reshape(self.batch, -1, self.cfg.hidden)
        if self.pos_embed is not None:
            x = x + self.pos_embed.index_select(0, pos_idx + 2)[None]
        return x

    def _sample(self, x_last):
        h = self._norm(x_last, self.final_norm_w, self.final_norm_b)
        self.last_hidden = h
        return self._pick(self._project(h))                                    # [B, vocab_local]

    def _project(self, h):
        """Vocabulary projection of this rank's slice: the library's dense GEMV for a decode batch, the framework's
        GEMM for more rows."""
        h = h.reshape(-1, self.cfg.hidden)
        if h.shape[0] <= 8:
            return ops.dense_gemv(h.contiguous(), self.lm_head)
        return h @ self.lm_head.t()

    def _pick(self, logits):
        logits = logits.float()
        pad = (self.rank + 1) * self.vocab_local - self.cfg.vocab   # padding columns of the last rank's slice
        if pad > 0:
            logits[:, self.vocab_local - pad:] = float("-inf")
        self.last_logits = logits
        val, idx = logits.max(dim=-1)
        idx = idx + self.rank * self.vocab_local
        if self.world > 1 and self.exchange is not None and logits.shape[0] <= 8:
            # every rank's best (logit, token) through the peer-memory exchange: a sum over ranks of vectors that are
            # zero outside the rank's own slots is a gather; the numbers travel as pairs of fp16 values that are
            # exact (logit = hi + lo, token = 256 * hi + lo)
            B = logits.shape[0]
            slots = torch.zeros((B, 4 * self.world), dtype=torch.float16, device=logits.device)
            hi = val.half()
            mine = slots[:, 4 * self.rank:4 * self.rank + 4]
            mine[:, 0] = hi
            mine[:, 1] = (val - hi.float()).half()
            mine[:, 2] = (idx // 256).half()
            mine[:, 3] = (idx % 256).half()
            ops.tp_allreduce(slots, self.exchange)
            got = slots.float().reshape(B, self.world, 4)
            best = (got[:, :, 0] + got[:, :, 1]).argmax(dim=1, keepdim=True)
            idx = (got[:, :, 2] * 256 + got[:, :, 3]).gather(1, best)[:, 0].long()
        elif self.world > 1:
            vals = [torch.empty_like(val) for _ in range(self.world)]
            idxs = [torch.empty_like(idx) for _ in range(self.world)]
            dist.all_gather(vals, val, group=self.group)
            dist.all_gather(idxs, idx, group=self.group)
            best = torch.stack(vals).argmax(dim=0)
            idx = torch.stack(idxs).gather(0, best[None])[0]
        return idx.clamp_(max=self.cfg.vocab - 1)

    # ---- public ----
    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor):
        """prompt: int64 [B, S]; fills the KV cache and leaves the first generated token in self.tokens."""
        B, S = prompt.shape
        check_positions(0, S, self.cfg.max_seq)
        self._pos_host = S
        pos_idx = torch.arange(S, device=self.device)
        x = self._embed(prompt, pos_idx)
        for L in self.layers:
            x = self._layer(L, x, pos_idx, S, decode=False)
        self.tokens.copy_(self._sample(x[:, -1]))
        self.pos.fill_(S)

    @torch.no_grad()
    def _decode_step(self):
        if self.fused:
            return self._decode_step_fused()
        x = self._embed(self.tokens, self.pos)
        for L in self.layers:
            x = self._layer(L, x, self.pos, 1, decode=True)
        self.tokens.copy_(self._sample(x[:, -1]))
        self.pos.add_(1)

    def _decode_step_fused(self):
        """One token per sequence with the fused helper kernels: per layer 5 small launches + 4 linears."""
        cfg, B = self.cfg, self.batch
        hd, rms = cfg.head_dim, cfg.arch == "llama"
        eps = 1e-6 if rms else 1e-5
        x = self._embed(self.tokens, self.pos).reshape(B, cfg.hidden).contiguous()
        h = torch.empty_like(x)
        delta = None   # output of the previous row-parallel linear, added to the residual by the next norm
        for L in self.layers:
            ops.add_norm(x, delta, L.norm1_w, L.norm1_b, h, eps, rms)
            qkv = L.qkv(h)
            att = torch.empty((B, L.heads_local * hd), dtype=torch.float16, device=self.device)
            # rotary embedding, cache write and single-query attention in one launch
            ops.attn_step(qkv, self.cos, self.sin, self.pos, L.k_cache, L.v_cache, att, L.heads_local, hd, rms)
            o = self._row(L.o, att)
            ops.add_norm(x, o, L.norm2_w, L.norm2_b, h, eps, rms)
            u = L.up(h)
            fold = _lib.ACT_SWIGLU if rms else _lib.ACT_RELU
            if self.fold_activation and isinstance(L.down, QuantLinear) and L.down.can_fold(B, fold):
                delta = self._row(L.down, u, fold)       # SiLU(gate) * up / ReLU inside the GEMV's read of x
            else:
                a = torch.empty((B, L.inter_local), dtype=torch.float16, device=self.device)
                ops.act(u, a, L.inter_local, rms)
                delta = self._row(L.down, a)
        ops.add_norm(x, delta, self.final_norm_w, self.final_norm_b, h, eps, rms)
        self.last_hidden = h
        logits = self._project(h)
        if (logits.dtype is torch.float16 and logits.is_contiguous()
                and (self.world == 1 or (self.exchange is not None and B <= 8))):   # the exchange takes up to 8 rows
            # greedy pick and the step's position in the library's kernels: one launch on one GPU, two around the
            # exchange on several (the framework's route is a dozen element-wise launches)
            self.last_logits = logits
            valid = min(self.vocab_local, self.cfg.vocab - self.rank * self.vocab_local)
            top = self.cfg.vocab - 1
            if self.world == 1:
                ops.pick_local(logits, valid, 0, 1, 0, None, self.tokens, top, self.pos)
            else:
                slots = torch.empty((B, 4 * self.world), dtype=torch.float16, device=self.device)
                ops.pick_local(logits, valid, self.rank * self.vocab_local, self.world, self.rank, slots, None, top)
                ops.tp_allreduce(slots, self.exchange)
                ops.pick_final(slots, self.world, self.tokens, top, self.pos)
        else:
            self.tokens.copy_(self._pick(logits))
            self.pos.add_(1)

    def capture(self):
        """Warm up (allocates scratch, builds run-time views) and capture one decode step in a CUDA graph."""
        check_positions(self._pos_host, 3, self.cfg.max_seq)   # two warm-up steps and the captured one
        saved_pos, saved_tok = self.pos.clone(), self.tokens.clone()
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._decode_step()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._decode_step()
        self.pos.copy_(saved_pos)
        self.tokens.copy_(saved_tok)

    #: work splits :meth:`tune` tries: (K slices per SM that the cluster size aims at, CTAs per SM that the footprint is
    #: sized for; 0 = the library's choice), ``None`` = the library's defaults for a GEMV on its own
    TUNINGS = (None, (2, 0), (4, 0), (6, 0), (2, 3))

    def tune(self, steps: int = 12, candidates=TUNINGS) -> dict:
        """Choose the GEMV work split of each kind of linear layer (qkv, o, up, down) by timing the captured decode
        step, one kind at a time with the others held.  This is the counterpart of the reference's per-shape tile
        tables (auto_gptq/nn_modules/tvm_untils/pycuda_warpper.py:77-127), measured in place because the best split
        depends on the kernels around the GEMV (4-5 % of a Llama-7B step, 2-3 % of an OPT-66B step on one B200).
        Position and tokens are restored; cache rows past the current position are used as scratch.  With several
        ranks every rank calls this at the same point and all take the split that is fastest for the slowest rank.
        Returns {kind: tuning}; a batch of more than 8 rows does not run GEMVs and is left alone."""
        kinds = ("qkv", "o", "up", "down")
        chosen = {k: getattr(self.layers[0], k).gemv_tuning for k in kinds}
        if self.batch > 8 or self._pos_host + steps + 3 > self.cfg.max_seq:
            return chosen
        dev = self.device

        def apply(kind, tuning):
            for L in self.layers:
                getattr(L, kind).gemv_tuning = tuning

        def step_ms() -> float:
            self.capture()
            saved = (self.pos.clone(), self.tokens.clone(), self._pos_host)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev)
            e0.record()
            self.decode(steps)
            e1.record()
            torch.cuda.synchronize(dev)
            self.pos.copy_(saved[0])
            self.tokens.copy_(saved[1])
            self._pos_host = saved[2]
            t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
            if self.world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            return float(t.item())

        for kind in kinds:
            if not isinstance(getattr(self.layers[0], kind), QuantLinear):
                continue
            times = []
            for cand in candidates:
                apply(kind, cand)
                times.append(step_ms())
            chosen[kind] = candidates[times.index(min(times))]
            apply(kind, chosen[kind])
        self.capture()
        return chosen

    def decode(self, steps: int) -> torch.Tensor:
        check_positions(self._pos_host, steps, self.cfg.max_seq)
        self._pos_host += steps
        out = torch.empty(steps, self.batch, dtype=torch.long, device=self.device)
        for i in range(steps):
            if self.graph is not None:
                self.graph.replay()
            else:
                self._decode_step()
            out[i].copy_(self.tokens)
        return out

    def step_kernels(self) -> dict:
        """Run one more decode step under the framework's activity tracer and return {kernel name: launches}: what one
        token launches on this rank (the evidence that a tensor-parallel step holds no library collective).  Not for
        timing."""
        import collections
        from torch.profiler import ProfilerActivity, profile
        torch.cuda.synchronize(self.device)
        if self._pos_host >= self.cfg.max_seq:     # the caches are full: trace a repeat of the last position
            self._pos_host -= 1
            self.pos.sub_(1)
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            self.decode(1)
            torch.cuda.synchronize(self.device)
        counts: dict = collections.Counter()
        for e in prof.events():
            if e.device_type == torch.autograd.DeviceType.CUDA:
                name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0]
                counts[name[:80]] += 1
        return dict(counts)

    def close(self) -> None:
        """Release the peer-memory exchange (every rank, after the last step has been synchronised)."""
        if self.exchange is not None:
            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
            self.exchange.close()
            self.exchange = None
            for L in self.layers:
                L.o.exchange = L.down.exchange = None

    def gather_logits(self) -> torch.Tensor:
        """The latest logits over the whole vocabulary ``[B, vocab]`` (every rank gets them)."""
        lg = self.last_logits
        if self.world > 1:
            parts = [torch.empty_like(lg) for _ in range(self.world)]
            dist.all_gather(parts, lg.contiguous(), group=self.group)
            lg = torch.cat(parts, dim=1)
        return lg[:, :self.cfg.vocab].float()

    def bytes_per_token(self) -> int:
        """Bytes of weights this rank streams per decode step (packed linears + its lm_head slice)."""
        return sum(L.linear_bytes() for L in self.layers) + self.lm_head.numel() * 2


@torch.no_grad()
def tp_parity(cfg: DecoderConfig, prompt: torch.Tensor, device, fused_allreduce: bool = False) -> dict:
    """Does the tensor-parallel model compute what the unsharded model computes?  Every rank of the default
    process group builds its shard and runs the prompt plus one decode step; rank 0 also builds the whole model
    and compares the logits over the full vocabulary.  The yardstick is the output contract of the path applied
    to the vocabulary projection: ``1e-2 * ||h||_2 * max|w|`` per logit, h the final hidden state.  Returns
    ``{max_abs_err, tol, ok}`` on rank 0 (``{}`` elsewhere)."""
    rank = dist.get_rank() if dist.is_initialized() else 0
    batch = prompt.shape[0]
    m = GPTQDecoder(cfg, batch=batch, device=device, fused_allreduce=fused_allreduce)
    m.prefill(prompt)
    lg_prompt = m.gather_logits()
    ref = None
    tok = torch.zeros(batch, dtype=torch.long, device=device)
    if rank == 0:
        ref = GPTQDecoder(cfg, batch=batch, device=device, single=True)
        ref.prefill(prompt)
        tok.copy_(ref.tokens)
    if dist.is_initialized():
        dist.broadcast(tok, src=0)
    m.tokens.copy_(tok)           # both models continue from the same token even if a near-tie picked differently
    m.decode(1)
    lg_step = m.gather_logits()
    m.close()
    if rank != 0:
        return {}
    ref_prompt = ref.last_logits[:, :cfg.vocab]
    h = ref.last_hidden.float()
    ref.decode(1)
    ref_step = ref.last_logits[:, :cfg.vocab]
    world = m.world
    wmax = float(ref.lm_head.float().abs().max())
    tol = 1e-2 * float(h.norm(dim=-1).min()) * wmax
    finite = torch.isfinite(ref_prompt) & torch.isfinite(ref_step)
    err = max(float(((lg_prompt - ref_prompt).abs() * finite).max()), float(((lg_step - ref_step).abs() * finite).max()))
    return {"max_abs_err": err, "tol": tol, "ok": bool(err <= tol), "world": world,
            "fused_allreduce": bool(fused_allreduce), "same_first_token": bool(torch.equal(m.tokens, ref.tokens))}
