"""The decoder on the fused compute+communication kernels: the on-demand engine without FSDP's hooks.

Same architecture and parameter names as :class:`odc_b200.models.DecoderLM`, but no parameter is an
``nn.Parameter`` and nothing is all-gathered ahead of use:

* the four projection matrices of every layer are :class:`ShardedParameter` s: forward pulls the
  owners' rows INSIDE the GEMM kernel (``gather_linear``), the input gradient pulls them again
  (``gather_dgrad``) or reuses the assembled weight (``keep_weight``), and the weight gradient is
  reduced into its owners from the GEMM epilogue (``wgrad_scatter``);
* the embedding / LM-head matrix is a ``ShardedParameter`` too; it is pulled once per microbatch into
  a reused buffer (the lookup and the chunked loss both read it) and its gradient - the loss's
  weight gradient plus the lookup's scatter-add - is accumulated in fp32 on the producing rank and
  pushed to the owners once per microbatch (or once per minibatch, see below) on the side stream;
* norm weights and biases form one small flat sharded group: pulled once per minibatch, gradients
  accumulated locally in fp32 and pushed once per minibatch.

The reference reaches the same two hot paths by patching FSDP2 (odc/fsdp/fsdp2.py:218-313 gather on
the unshard path, 607-742 reduction on the backward path); the minibatch protocol is the same:
``start_minibatch`` (collective) ... any number of microbatches, different per rank ...
``finish_minibatch`` (collective) ... ``optimizer.step()``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import ops
from ..models.llama import DecoderConfig, DecoderLM
from ..ops import reference as ref
from ..primitives import GatherService
from ..runtime import control
from ..runtime.registry import SymmBufferRegistry
from . import linear as L
from .linear import OdcLinear, ShardedParameter


class SmallGroup:
    """Norm weights and biases: one flat vector, sharded evenly, pulled once per minibatch."""

    def __init__(self, named: Dict[str, torch.Tensor], pg, device, lowp_dtype):
        reg = SymmBufferRegistry.get_instance()
        self.pg = pg
        self.ranks = control.group_ranks(pg)
        self.world = len(self.ranks)
        self.index = self.ranks.index(control.rank())
        self.slots: Dict[str, tuple] = {}
        off = 0
        for name, t in named.items():
            self.slots[name] = (off, t.numel())
            off += (t.numel() + 7) // 8 * 8          # every parameter starts on a 16-byte boundary
        self.numel = off
        self.shard = ((off + self.world - 1) // self.world + 7) // 8 * 8
        flat = torch.zeros(self.shard * self.world, dtype=torch.float32, device=device)
        for name, t in named.items():
            o, n = self.slots[name]
            flat[o:o + n].copy_(t.reshape(-1))
        self.master = flat[self.index * self.shard:(self.index + 1) * self.shard].clone()
        self.lowp = reg.allocate_symm_buffer("odc_small_lowp", (self.shard,), lowp_dtype)
        self.lowp.copy_(self.master)
        self.key = "odc_small"
        self.acc = L._service().register(self.key, self.shard, torch.float32, pg)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.full = torch.zeros(self.shard * self.world, dtype=lowp_dtype, device=device, requires_grad=True)
        self.grad32 = torch.zeros(self.shard * self.world, dtype=torch.float32, device=device)
        self.grad_scale = 1.0 / (self.world * L.replicas())
        self.dirty = False
        self.full.register_post_accumulate_grad_hook(self._fold)

    def _fold(self, leaf):
        # one low-precision gradient per backward pass; the running sum over microbatches is kept in fp32
        self.grad32.add_(leaf.grad)
        leaf.grad = None
        self.dirty = True

    def view(self, name: str, shape) -> torch.Tensor:
        o, n = self.slots[name]
        return self.full[o:o + n].view(shape)

    def flat(self):
        return self.master, self.acc, self.m, self.v, self.lowp

    @torch.no_grad()
    def refresh(self, gather: GatherService) -> None:
        gather.gather_ranks(self.full.detach(), self.lowp, self.ranks)

    def push(self) -> None:
        if self.dirty:
            L._service().scatter_accumulate(self.key, self.grad32, self.pg, scale=self.grad_scale)
            self.grad32.zero_()
            self.dirty = False

    def _all(self, t: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(t) for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(parts, t.contiguous(), group=self.pg)
        else:
            parts[0] = t
        return torch.cat(parts)

    def load_flat(self, dst: torch.Tensor, named: Dict[str, torch.Tensor]) -> None:
        flat = torch.zeros(self.shard * self.world, dtype=torch.float32, device=dst.device)
        for name, t in named.items():
            o, n = self.slots[name]
            flat[o:o + n].copy_(t.reshape(-1))
        dst.copy_(flat[self.index * self.shard:(self.index + 1) * self.shard])


class _Embedding(torch.autograd.Function):
    """Lookup in the gathered matrix; backward scatter-adds into the producing rank's fp32 buffer and (with
    synchronisation on) pushes that buffer to the owners.  ``anchor`` only makes autograd call backward."""

    @staticmethod
    def forward(ctx, ids, anchor, model):
        ctx.model = model
        ctx.save_for_backward(ids)
        p = model.embed
        return F.embedding(ids, model.embed_full[:p.out_features])

    @staticmethod
    def backward(ctx, dx):
        model = ctx.model
        (ids,) = ctx.saved_tensors
        p = model.embed
        p.wait_push()
        buf = p.local_buffer()
        buf.index_add_(0, ids.reshape(-1), dx.reshape(-1, dx.shape[-1]).float())
        p.local_dirty = True
        if L.requires_gradient_sync():
            p.push_local(side_stream=True)   # overlaps the next microbatch's forward
        return None, None, None


class _FusedLinearCrossEntropy(torch.autograd.Function):
    """Chunked loss against the gathered LM-head matrix (same mathematics as ``ops.linear_cross_entropy``;
    the reference's chunked head is examples/llm_training/lm_head.py:7-59).  The weight gradient goes to the
    producing rank's fp32 buffer instead of to autograd."""

    @staticmethod
    def forward(ctx, h, labels, loss_scale, model, ignore_index, chunk):
        p = model.head_param()
        w = model.head_full()[:p.out_features]
        if h.is_cuda:
            T, H = h.shape
            ext = ops._ext()
            dh = torch.empty_like(h)
            dw32 = torch.empty(p.out_features, H, dtype=torch.float32, device=h.device)  # written by the first chunk
            loss = torch.zeros((), dtype=torch.float32, device=h.device)
            logits = torch.empty(min(chunk, T), p.out_features, dtype=torch.bfloat16, device=h.device)
            if T == 0:
                dw32.zero_()
            for s in range(0, T, chunk):
                e = min(T, s + chunk)
                lg = logits[: e - s]
                ops.gemm(h[s:e], w, "nt", out=lg)
                ext.ce_fwd_bwd(lg, labels[s:e], None if loss_scale is None else loss_scale[s:e], loss, ignore_index)
                ops._count()
                ops.gemm(lg, w, "nn", out=dh[s:e])
                ops.gemm(lg, h[s:e], "tn", out=dw32, accumulate=s > 0)
        else:
            with torch.enable_grad():
                h_ = h.detach().requires_grad_()
                w_ = w.detach().float().requires_grad_()
                loss = ref.linear_cross_entropy(h_, w_, labels, loss_scale, ignore_index, chunk)
                dh, dw32 = torch.autograd.grad(loss, [h_, w_])
            loss = loss.detach()
        ctx.save_for_backward(dh, dw32)
        ctx.model = model
        return loss

    @staticmethod
    def backward(ctx, dloss):
        dh, dw32 = ctx.saved_tensors
        model = ctx.model
        p = model.head_param()
        p.wait_push()
        buf = p.local_buffer()
        buf[:p.out_features].addcmul_(dw32, dloss.to(dw32.dtype))
        p.local_dirty = True
        if p is not model.embed and L.requires_gradient_sync():
            p.push_local(side_stream=True)   # a tied matrix is pushed by the lookup's backward, which runs last
        return dh * dloss.to(dh.dtype), None, None, None, None, None


class _FusedTokenLogProbs(torch.autograd.Function):
    """Per-token log-probabilities against the gathered LM-head matrix (``ops.linear_token_logprobs`` with the
    weight gradient going to the producing rank's fp32 buffer; the reference's policy-gradient head is
    examples/llm_training/lm_head.py:62-190).  Backward recomputes the chunks' logits."""

    @staticmethod
    def forward(ctx, h, ids, model, temperature, ignore_index, chunk):
        p = model.head_param()
        w = model.head_full()[:p.out_features]
        ctx.save_for_backward(h, ids)
        ctx.model, ctx.args = model, (temperature, ignore_index, chunk)
        with torch.no_grad():
            return ops.linear_token_logprobs(h, w, ids, temperature, ignore_index, chunk)

    @staticmethod
    def backward(ctx, dlogp):
        h, ids = ctx.saved_tensors
        model = ctx.model
        temperature, ignore_index, chunk = ctx.args
        p = model.head_param()
        w = model.head_full()[:p.out_features]
        with torch.enable_grad():
            h_ = h.detach().requires_grad_()
            w_ = w.detach().requires_grad_()
            lp = ops.linear_token_logprobs(h_, w_, ids, temperature, ignore_index, chunk)
            dh, dw = torch.autograd.grad(lp, [h_, w_], dlogp)
        p.wait_push()
        buf = p.local_buffer()
        buf[:p.out_features].add_(dw)
        p.local_dirty = True
        if p is not model.embed and L.requires_gradient_sync():
            p.push_local(side_stream=True)
        return dh, None, None, None, None, None


class FusedDecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, i: int, src, small: SmallGroup, pg, keep_weight, lowp_dtype):
        super().__init__()
        self.cfg, self.small, self.i = cfg, small, i
        mk = lambda name, w: OdcLinear(w.shape[1], w.shape[0], pg=pg, name=f"L{i}_{name}", keep_weight=keep_weight,
                                       full=w, lowp_dtype=lowp_dtype)
        self.wqkv = mk("wqkv", src.attn.wqkv.data)
        self.wo = mk("wo", src.attn.wo.data)
        self.w_gate_up = mk("w_gate_up", src.mlp.w_gate_up.data)
        self.w_down = mk("w_down", src.mlp.w_down.data)

    def forward(self, x, position_ids, cu_seqlens, max_seqlen):
        c, s, i = self.cfg, self.small, self.i
        T = x.shape[0]
        h, x = ops.rms_norm_residual(x, s.view(f"layers.{i}.attn_norm.weight", (c.hidden_size,)), c.rms_eps)
        bias = s.view(f"layers.{i}.attn.bqkv", (c.qkv_dim,)) if c.qkv_bias else None
        qkv = self.wqkv(h, bias=bias)
        qkv = ops.rope_qkv(qkv, position_ids, c.num_heads, c.num_kv_heads, c.head_dim, c.rope_theta,
                           c.rope_inv_freq(qkv.device))
        o = ops.varlen_attention_qkv(qkv, c.num_heads, c.num_kv_heads, c.head_dim, cu_seqlens, max_seqlen, causal=True)
        x = self.wo(o.reshape(T, c.num_heads * c.head_dim), residual=x)
        h, x = ops.rms_norm_residual(x, s.view(f"layers.{i}.mlp_norm.weight", (c.hidden_size,)), c.rms_eps)
        return self.w_down(ops.swiglu(self.w_gate_up(h)), residual=x)


class FusedDecoderLM(nn.Module):
    """``DecoderLM`` with every matrix sharded by rows and every matrix product fused with its transfer."""

    def __init__(self, cfg: DecoderConfig, device=None, seed: Optional[int] = 0, pg=None, keep_weight: bool = False,
                 lowp_dtype: Optional[torch.dtype] = None, source: Optional[DecoderLM] = None, replicate_pg=None,
                 mesh=None):
        """``pg``: the group the rows are sharded over (default: all ranks).  ``replicate_pg``: hybrid sharding, the
        ranks that hold the same rows as this one; or pass a 2-D ``mesh`` with dimensions
        ``("dp_replicate", "dp_shard")`` as for ``fully_shard``."""
        super().__init__()
        if mesh is not None:
            pg, replicate_pg = mesh.get_group("dp_shard"), mesh.get_group("dp_replicate")
        L.set_replicate_group(replicate_pg)
        reg = SymmBufferRegistry.get_instance()
        device = torch.device(device) if device is not None else reg.heap.device
        if lowp_dtype is None:
            lowp_dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
        self.cfg, self.pg, self.device, self.lowp_dtype = cfg, pg, device, lowp_dtype
        if source is None:   # the same initial weights as DecoderLM(cfg).reset_parameters(seed) gives every engine
            with torch.device(device):
                source = DecoderLM(cfg)
            source.reset_parameters(seed=seed)
        small = {}
        for i, layer in enumerate(source.layers):
            small[f"layers.{i}.attn_norm.weight"] = layer.attn_norm.weight.data
            small[f"layers.{i}.mlp_norm.weight"] = layer.mlp_norm.weight.data
            if cfg.qkv_bias:
                small[f"layers.{i}.attn.bqkv"] = layer.attn.bqkv.data
        small["norm.weight"] = source.norm.weight.data
        self.gather = GatherService()
        self.small = SmallGroup(small, pg, device, lowp_dtype)
        self.layers = nn.ModuleList([FusedDecoderLayer(cfg, i, layer, self.small, pg, keep_weight, lowp_dtype)
                                     for i, layer in enumerate(source.layers)])
        self.embed = ShardedParameter("embed", tuple(source.embed.weight.shape), pg, device, full=source.embed.weight.data,
                                      lowp_dtype=lowp_dtype)
        self.lm_head = None
        if source.lm_head is not None:
            self.lm_head = ShardedParameter("lm_head", tuple(source.lm_head.shape), pg, device, full=source.lm_head.data,
                                            lowp_dtype=lowp_dtype)
        self.embed_full = torch.empty(self.embed.world * self.embed.rows_per_rank, cfg.hidden_size, dtype=lowp_dtype,
                                      device=device)
        self.lm_head_full = None if self.lm_head is None else torch.empty(
            self.lm_head.world * self.lm_head.rows_per_rank, cfg.hidden_size, dtype=lowp_dtype, device=device)
        self._head_fresh = False
        del source

    # -- parameters ------------------------------------------------------------------------------------
    def head_param(self) -> ShardedParameter:
        return self.embed if self.lm_head is None else self.lm_head

    def head_full(self) -> torch.Tensor:
        return self.embed_full if self.lm_head is None else self.lm_head_full

    def matrices(self) -> Dict[str, ShardedParameter]:
        out = {"embed.weight": self.embed}
        for i, layer in enumerate(self.layers):
            out[f"layers.{i}.attn.wqkv"] = layer.wqkv.weight
            out[f"layers.{i}.attn.wo"] = layer.wo.weight
            out[f"layers.{i}.mlp.w_gate_up"] = layer.w_gate_up.weight
            out[f"layers.{i}.mlp.w_down"] = layer.w_down.weight
        if self.lm_head is not None:
            out["lm_head"] = self.lm_head
        return out

    def optimizer_groups(self) -> List:
        return list(self.matrices().values()) + [self.small]

    # -- minibatch protocol -----------------------------------------------------------------------------
    @torch.no_grad()
    def start_minibatch(self) -> None:
        """Zero the accumulators, publish this rank's freshly updated rows, pull the small group (collective)."""
        L.set_requires_gradient_sync(True)
        L.start_minibatch()
        self.small.refresh(self.gather)

    def set_requires_gradient_sync(self, flag: bool) -> None:
        L.set_requires_gradient_sync(flag)

    @torch.no_grad()
    def finish_minibatch(self) -> None:
        """Push what is still held locally and wait for every contribution to this rank's rows (collective)."""
        self.small.push()
        L.finish_minibatch(optimizer_step=False)

    def transport_launches(self) -> int:
        return getattr(L._service().transport, "launches", 0) + getattr(self.gather.transport, "launches", 0)

    def stop(self) -> None:
        L._service().stop()
        L.reset()
        from .. import finalize_distributed
        finalize_distributed()

    # -- forward ------------------------------------------------------------------------------------------
    def hidden_states(self, input_ids, position_ids, cu_seqlens, max_seqlen):
        with torch.no_grad():
            # one pull per microbatch, like a root FSDP unit that stays unsharded from forward to backward
            self.gather.gather_ranks(self.embed_full, self.embed.lowp, self.embed.ranks)
            if self.lm_head is not None:
                self.gather.gather_ranks(self.lm_head_full, self.lm_head.lowp, self.lm_head.ranks)
        x = _Embedding.apply(input_ids, self.small.full, self)
        for layer in self.layers:
            if self.cfg.activation_checkpointing and torch.is_grad_enabled():
                x = checkpoint(layer, x, position_ids, cu_seqlens, max_seqlen, use_reentrant=False)
            else:
                x = layer(x, position_ids, cu_seqlens, max_seqlen)
        return ops.rms_norm(x, self.small.view("norm.weight", (self.cfg.hidden_size,)), self.cfg.rms_eps)

    def forward(self, input_ids, position_ids, cu_seqlens, max_seqlen, labels=None, loss_scale=None,
                return_logprobs: bool = False, temperature: float = 1.0):
        """Same contract as ``DecoderLM.forward``: hidden states, the summed weighted loss, or (``return_logprobs``)
        the per-token log-probabilities of ``labels``."""
        h = self.hidden_states(input_ids, position_ids, cu_seqlens, max_seqlen)
        if labels is None:
            return h
        if return_logprobs:
            return _FusedTokenLogProbs.apply(h.contiguous(), labels.contiguous(), self, float(temperature), -100,
                                             self.cfg.ce_chunk)
        if loss_scale is not None and loss_scale.dtype != torch.float32:
            loss_scale = loss_scale.float()
        return _FusedLinearCrossEntropy.apply(h.contiguous(), labels.contiguous(), loss_scale, self, -100,
                                              self.cfg.ce_chunk)

    @torch.no_grad()
    def logits(self, input_ids, position_ids, cu_seqlens, max_seqlen):
        """``[T, vocab]`` logits (inference helper; pulls the head matrix like a forward pass does)."""
        h = self.hidden_states(input_ids, position_ids, cu_seqlens, max_seqlen)
        p = self.head_param()
        return ops.linear(h, self.head_full()[:p.out_features])

    # -- whole-model state (collective): the names and shapes DecoderLM.state_dict() has ------------------
    @torch.no_grad()
    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        out = {name: p.full_master() for name, p in self.matrices().items()}
        flat = self.small._all(self.small.master)
        for name, (o, n) in self.small.slots.items():
            out[name] = flat[o:o + n].clone()
        return out

    @torch.no_grad()
    def load_full_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for name, p in self.matrices().items():
            p.load_full(sd[name].to(p.master.device, torch.float32))
        self.small.load_flat(self.small.master, {n: sd[n].to(self.device, torch.float32) for n in self.small.slots})
        self.small.lowp.copy_(self.small.master)


class FusedOptimizer:
    """AdamW over the rows this rank owns, straight from the accumulators the peers pushed into.

    One kernel per matrix updates the fp32 master rows and moments and writes the low-precision rows the
    peers will pull in the next minibatch; the gradient-norm clip is folded in as a scale.  Takes the place
    of ``torch.optim.AdamW`` over DTensor shards (examples/llm_training/torch_fsdp2.py:322, 441-448).
    """

    def __init__(self, model: FusedDecoderLM, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01):
        self.model, self.lr, self.betas, self.eps, self.weight_decay = model, lr, betas, eps, weight_decay
        self.step_count = 0
        self._clip_scale = 1.0

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float) -> torch.Tensor:
        groups = self.model.optimizer_groups()
        dev = self.model.device
        total = torch.zeros((), dtype=torch.float32, device=dev)
        for g in groups:
            acc = g.flat()[1]
            if acc.is_cuda:
                part = torch.zeros((), dtype=torch.float32, device=dev)
                ops._ext().sumsq(acc, part)
                total += part
            else:
                total += acc.float().pow(2).sum()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(total, group=self.model.pg)   # rows are disjoint across the group
        norm = total.sqrt()
        self._clip_scale = float(min(1.0, max_norm / (float(norm) + 1e-6)))
        return norm

    @torch.no_grad()
    def step(self) -> None:
        self.step_count += 1
        for g in self.model.optimizer_groups():
            master, acc, m, v, lowp = g.flat()
            ops.fused_adamw_(master, acc, m, v, lowp, self.lr, self.betas[0], self.betas[1], self.eps,
                             self.weight_decay, self.step_count, self._clip_scale)
        self._clip_scale = 1.0

    def zero_grad(self, set_to_none: bool = True) -> None:
        pass  # gradients live in the accumulators, which start_minibatch clears

    @torch.no_grad()
    def full_state_dict(self) -> Dict:
        """``{"step", "exp_avg": {name: tensor}, "exp_avg_sq": {...}}`` with whole tensors (collective)."""
        m, v = {}, {}
        for name, p in self.model.matrices().items():
            m[name], v[name] = p._full_of(p.m), p._full_of(p.v)
        s = self.model.small
        fm, fv = s._all(s.m), s._all(s.v)
        for name, (o, n) in s.slots.items():
            m[name], v[name] = fm[o:o + n].clone(), fv[o:o + n].clone()
        return {"step": self.step_count, "exp_avg": m, "exp_avg_sq": v}

    @torch.no_grad()
    def load_full_state_dict(self, sd: Dict) -> None:
        if "exp_avg" not in sd:   # the layout a full torch.optim.AdamW state dict has (state by parameter name)
            st = sd["state"]
            sd = {"step": max((int(float(e["step"])) for e in st.values()), default=0),
                  "exp_avg": {k: e["exp_avg"] for k, e in st.items()},
                  "exp_avg_sq": {k: e["exp_avg_sq"] for k, e in st.items()}}
        self.step_count = int(sd["step"])
        for name, p in self.model.matrices().items():
            dev = p.master.device
            p.load_full(p.full_master(), sd["exp_avg"][name].to(dev), sd["exp_avg_sq"][name].to(dev))
        s = self.model.small
        s.load_flat(s.m, {n: sd["exp_avg"][n].to(s.m.device) for n in s.slots})
        s.load_flat(s.v, {n: sd["exp_avg_sq"][n].to(s.v.device) for n in s.slots})
