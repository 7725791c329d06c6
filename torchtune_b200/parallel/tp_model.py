"""Tensor-parallel form of a dense Llama-style decoder.

:func:`tensor_parallelize` rewrites a resident :class:`~torchtune_b200.modules.TransformerDecoder` in place
(same layer layout as the reference's Llama-3 plan, torchtune/models/llama3/_parallelism.py:19-130):

* the residual stream is sharded by token rows (``batch·seq / tp`` rows per rank) — norms, residual adds,
  embedding lookup and the loss run on the shard;
* ``q/k/v`` are one fused column-parallel projection (all-gather → GEMM kernel), attention runs on the local
  heads over full sequences, ``output_proj`` is row-parallel (GEMM → reduce-scatter kernel with the residual
  add fused into the reduction);
* ``w1/w3`` are one fused column-parallel projection, ``w2`` row-parallel;
* norm scales, embeddings and the output head stay replicated; their gradients are summed over the group
  before the optimizer step (:meth:`TPDecoder.sync_replicated_grads`).

``full_state_dict`` / ``load_full_state_dict`` translate between the sharded parameters and the ordinary
checkpoint layout (``layers.N.attn.q_proj.weight`` …).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
from torch import nn

from .. import ops
from ..modules import TransformerDecoder, TransformerSelfAttentionLayer
from ..modules.attention import _as_mask
from .tp import TensorParallelContext, column_parallel_linear, row_parallel_linear


def _rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n : (rank + 1) * n]


def _wants_fp8(projs, what: str) -> bool:
    """``True`` when every projection is an fp8-training linear (tensorwise scaling: the only recipe that combines with tensor
    parallelism, as in the reference, torchtune/training/quantization.py:277), ``False`` when all are plain linears."""
    kinds = {type(p).__name__ for p in projs}
    if any(p is None or p.bias is not None for p in projs) or not kinds <= {"Linear", "Float8Linear"}:
        raise NotImplementedError(f"tensor parallelism supports bias-free, un-adapted {what}")
    if kinds == {"Linear"}:
        return False
    if kinds != {"Float8Linear"}:
        raise NotImplementedError(f"tensor parallelism needs all {what} in the same precision")
    if any(getattr(p, "recipe", "tensorwise") != "tensorwise" for p in projs):
        raise ValueError("fp8 training with tensor parallelism supports only tensorwise scaling")
    return True


def _fp8_matmul(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with dynamically scaled fp8 operands, one scale per tensor — here per *shard*: every rank scales the slice of
    the weight it owns, a finer granularity than one scale for the whole matrix."""
    y = ops.fp8_linear(x, w)
    if y is None:
        from ..training.quantization import _fp8_roundtrip

        y = ops.linear(_fp8_roundtrip(x, None), _fp8_roundtrip(w, None))
    return y


def _column(x_shard: torch.Tensor, w: torch.Tensor, tp: TensorParallelContext, fp8: bool) -> torch.Tensor:
    if fp8:  # NCCL gather + fp8 tensor-core GEMM (the fused gather → GEMM kernel is bf16)
        return _fp8_matmul(_GatherRows.apply(x_shard, tp), w)
    return column_parallel_linear(x_shard, w, tp)


def _row(x: torch.Tensor, w: torch.Tensor, tp: TensorParallelContext, residual: torch.Tensor, fp8: bool) -> torch.Tensor:
    if fp8:
        return residual + _ScatterSumRows.apply(_fp8_matmul(x, w), tp)
    return row_parallel_linear(x, w, tp, residual)


class TPAttention(nn.Module):
    def __init__(self, attn: nn.Module, tp: TensorParallelContext):
        super().__init__()
        w, r = tp.world, tp.rank
        if attn.num_heads % w or attn.num_kv_heads % w:
            raise ValueError(f"tensor parallel size {w} must divide num_heads ({attn.num_heads}) and num_kv_heads ({attn.num_kv_heads})")
        self.fp8 = _wants_fp8((attn.q_proj, attn.k_proj, attn.v_proj, attn.output_proj), "attention projections")
        self.tp = tp
        self.head_dim = attn.head_dim
        self.heads, self.kv_heads = attn.num_heads // w, attn.num_kv_heads // w
        self.full_heads, self.full_kv_heads = attn.num_heads, attn.num_kv_heads
        hd = self.head_dim
        q = attn.q_proj.weight.data[r * self.heads * hd : (r + 1) * self.heads * hd]
        k = attn.k_proj.weight.data[r * self.kv_heads * hd : (r + 1) * self.kv_heads * hd]
        v = attn.v_proj.weight.data[r * self.kv_heads * hd : (r + 1) * self.kv_heads * hd]
        self.wqkv = nn.Parameter(torch.cat([q, k, v]).contiguous())
        in_per = attn.output_proj.weight.shape[1] // w
        self.wo = nn.Parameter(attn.output_proj.weight.data[:, r * in_per : (r + 1) * in_per].contiguous())
        self.pos_embeddings, self.q_norm, self.k_norm = attn.pos_embeddings, attn.q_norm, attn.k_norm
        self.qk_norm_before_rope = getattr(attn, "qk_norm_before_rope", False)
        self.is_causal, self.scale, self.softcap = attn.is_causal, attn.scale, attn.softcap

    def _pos(self, t: torch.Tensor, norm: Optional[nn.Module], input_pos) -> torch.Tensor:
        if norm is not None and self.qk_norm_before_rope:
            t = norm(t)
        if self.pos_embeddings is not None:
            t = self.pos_embeddings(t, input_pos=input_pos)
        if norm is not None and not self.qk_norm_before_rope:
            t = norm(t)
        return t

    def forward(self, hn: torch.Tensor, residual: torch.Tensor, b: int, s: int, mask, input_pos) -> torch.Tensor:
        hd = self.head_dim
        qkv = _column(hn, self.wqkv, self.tp, self.fp8)  # [b·s, (h + 2·h_kv)·hd] for the local heads
        nq, nk = self.heads * hd, self.kv_heads * hd
        q = self._pos(qkv[:, :nq].reshape(b, s, self.heads, hd), self.q_norm, input_pos)
        k = self._pos(qkv[:, nq : nq + nk].reshape(b, s, self.kv_heads, hd), self.k_norm, input_pos)
        v = qkv[:, nq + nk :].reshape(b, s, self.kv_heads, hd)
        out = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), _as_mask(mask, default_causal=self.is_causal and mask is None), scale=self.scale, softcap=self.softcap)
        return _row(out.reshape(b * s, nq), self.wo, self.tp, residual, self.fp8)

    # inference (replicated activations, local-head KV cache) -------------------------------
    def setup_cache(self, batch_size: int, dtype: torch.dtype, max_seq_len: int) -> None:
        from ..modules import KVCache

        self.kv_cache = KVCache(batch_size=batch_size, max_seq_len=max_seq_len, num_kv_heads=self.kv_heads, head_dim=self.head_dim, dtype=dtype)

    def forward_replicated(self, hn: torch.Tensor, mask, input_pos) -> torch.Tensor:
        """``hn``: ``[b, s, d]`` identical on every rank → this rank's partial ``[b, s, d]`` of the attention output projection
        (the caller sums the partials over the group)."""
        b, s, _ = hn.shape
        hd = self.head_dim
        qkv = ops.linear(hn, self.wqkv)
        nq, nk = self.heads * hd, self.kv_heads * hd
        q = self._pos(qkv[..., :nq].reshape(b, s, self.heads, hd), self.q_norm, input_pos)
        k = self._pos(qkv[..., nq : nq + nk].reshape(b, s, self.kv_heads, hd), self.k_norm, input_pos)
        v = qkv[..., nq + nk :].reshape(b, s, self.kv_heads, hd)
        cache = getattr(self, "kv_cache", None)
        if cache is not None:
            k, v = cache.update(k.contiguous(), v.contiguous())
        attn_mask = _as_mask(mask, default_causal=self.is_causal and mask is None and cache is None)
        out = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), attn_mask, scale=self.scale, softcap=self.softcap)
        return ops.linear(out.reshape(b, s, nq), self.wo)

    # checkpoint layout ----------------------------------------------------------------------
    def gather_full(self, prefix: str) -> Dict[str, torch.Tensor]:
        tp, hd = self.tp, self.head_dim
        nq, nk = self.heads * hd, self.kv_heads * hd
        w = self.wqkv.data
        return {
            f"{prefix}q_proj.weight": tp.all_gather_rows(w[:nq].contiguous()),
            f"{prefix}k_proj.weight": tp.all_gather_rows(w[nq : nq + nk].contiguous()),
            f"{prefix}v_proj.weight": tp.all_gather_rows(w[nq + nk :].contiguous()),
            f"{prefix}output_proj.weight": tp.all_gather_rows(self.wo.data.t().contiguous()).t().contiguous(),
        }


class TPMLP(nn.Module):
    def __init__(self, mlp: nn.Module, tp: TensorParallelContext):
        super().__init__()
        w, r = tp.world, tp.rank
        self.fp8 = _wants_fp8((mlp.w1, mlp.w2, mlp.w3), "gated MLP projections")
        if not isinstance(mlp.activation, nn.SiLU):
            raise NotImplementedError("tensor parallelism supports SwiGLU MLPs")
        hidden = mlp.w1.weight.shape[0]
        if hidden % w:
            raise ValueError(f"tensor parallel size {w} must divide the MLP width {hidden}")
        per = hidden // w
        self.tp, self.per = tp, per
        self.w13 = nn.Parameter(torch.cat([mlp.w1.weight.data[r * per : (r + 1) * per], mlp.w3.weight.data[r * per : (r + 1) * per]]).contiguous())
        self.w2 = nn.Parameter(mlp.w2.weight.data[:, r * per : (r + 1) * per].contiguous())

    def forward(self, hn: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        gu = _column(hn, self.w13, self.tp, self.fp8)
        h = ops.swiglu(gu[:, : self.per].contiguous(), gu[:, self.per :].contiguous())
        return _row(h, self.w2, self.tp, residual, self.fp8)

    def forward_replicated(self, hn: torch.Tensor) -> torch.Tensor:
        gu = ops.linear(hn, self.w13)
        h = ops.swiglu(gu[..., : self.per].contiguous(), gu[..., self.per :].contiguous())
        return ops.linear(h, self.w2)

    def gather_full(self, prefix: str) -> Dict[str, torch.Tensor]:
        tp = self.tp
        return {
            f"{prefix}w1.weight": tp.all_gather_rows(self.w13.data[: self.per].contiguous()),
            f"{prefix}w3.weight": tp.all_gather_rows(self.w13.data[self.per :].contiguous()),
            f"{prefix}w2.weight": tp.all_gather_rows(self.w2.data.t().contiguous()).t().contiguous(),
        }


class _GatherRows(torch.autograd.Function):
    """Sequence-sharded rows → all rows (backward: sum over ranks, keep own rows)."""

    @staticmethod
    def forward(ctx, x, tp: TensorParallelContext):
        ctx.tp = tp
        return tp.all_gather_rows(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.reduce_scatter_rows(g.contiguous()), None


class _ScatterSumRows(torch.autograd.Function):
    """Per-rank partial results for all rows → summed rows of this rank (backward: all-gather)."""

    @staticmethod
    def forward(ctx, x, tp: TensorParallelContext):
        ctx.tp = tp
        return tp.reduce_scatter_rows(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_gather_rows(g.contiguous()), None


class TPMoE(nn.Module):
    """Expert tensor parallelism (reference plan: torchtune/modules/moe/_parallelism.py:26-93 and
    torchtune/models/llama4/_parallelism.py:77-92): every rank holds all experts but only ``hidden / tp`` of each expert's
    width (``gate_proj`` / ``up_proj`` split on their last dimension, ``down_proj`` on its first); router and routing are
    replicated, so every rank routes the gathered tokens identically and produces a partial sum of the layer output that is
    reduce-scattered back to sequence-sharded rows.  The shared expert is split the same way."""

    def __init__(self, moe: nn.Module, tp: TensorParallelContext):
        super().__init__()
        from ..modules.moe import GroupedExperts

        src = moe.experts
        if not isinstance(src, GroupedExperts):
            raise NotImplementedError("tensor parallelism supports un-adapted grouped experts")
        w, r = tp.world, tp.rank
        if src.hidden_dim % w:
            raise ValueError(f"tensor parallel size {w} must divide the expert width {src.hidden_dim}")
        per = src.hidden_dim // w
        self.tp = tp
        self.router = moe.router
        local = GroupedExperts(dim=src.dim, hidden_dim=per, num_experts=src.num_experts, activation=src.act_fn)
        local.gate_proj = nn.Parameter(src.gate_proj.data[:, :, r * per : (r + 1) * per].contiguous())
        local.up_proj = nn.Parameter(src.up_proj.data[:, :, r * per : (r + 1) * per].contiguous())
        local.down_proj = nn.Parameter(src.down_proj.data[:, r * per : (r + 1) * per, :].contiguous())
        self.experts = local
        self.shared_expert = TPMLP(moe.shared_expert, tp) if moe.shared_expert is not None else None

    def _partial(self, flat: torch.Tensor) -> torch.Tensor:
        scores, token_idx, counts = self.router(flat)
        routed = self.experts(flat.index_select(0, token_idx) * scores.reshape(-1, 1), counts)
        out = self.shared_expert.forward_replicated(flat) if self.shared_expert is not None else torch.zeros_like(flat)
        return out.index_add(0, token_idx, routed.to(out.dtype))

    def forward(self, hn: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        full = _GatherRows.apply(hn, self.tp)
        return _ScatterSumRows.apply(self._partial(full), self.tp) + residual

    def forward_replicated(self, hn: torch.Tensor) -> torch.Tensor:
        return self._partial(hn.reshape(-1, hn.shape[-1])).reshape(hn.shape)

    def replicated_parameters(self) -> List[nn.Parameter]:
        return list(self.router.parameters())

    def gather_full(self, prefix: str) -> Dict[str, torch.Tensor]:
        tp = self.tp

        def cat(t: torch.Tensor, dim: int) -> torch.Tensor:  # gather along `dim` through the row gather
            moved = t.movedim(dim, 0).contiguous()
            return tp.all_gather_rows(moved).movedim(0, dim).contiguous()

        out = {f"{prefix}router.{k}": v.detach() for k, v in self.router.state_dict().items()}
        out[f"{prefix}experts.gate_proj"] = cat(self.experts.gate_proj.data, 2)
        out[f"{prefix}experts.up_proj"] = cat(self.experts.up_proj.data, 2)
        out[f"{prefix}experts.down_proj"] = cat(self.experts.down_proj.data, 1)
        if self.shared_expert is not None:
            out.update(self.shared_expert.gather_full(f"{prefix}shared_expert."))
        return out


class TPLayer(nn.Module):
    def __init__(self, layer: TransformerSelfAttentionLayer, tp: TensorParallelContext):
        super().__init__()
        if not isinstance(layer.sa_scale, nn.Identity) or not isinstance(layer.mlp_scale, nn.Identity):
            raise NotImplementedError("tensor parallelism does not support post-norm / gated residual layers")
        from ..modules.moe import MoE

        self.attn = TPAttention(layer.attn, tp)
        self.mlp = TPMoE(layer.mlp, tp) if isinstance(layer.mlp, MoE) else TPMLP(layer.mlp, tp)
        self.sa_norm, self.mlp_norm = layer.sa_norm, layer.mlp_norm
        self.mask_mod = layer.mask_mod

    def forward(self, h: torch.Tensor, b: int, s: int, mask, input_pos) -> torch.Tensor:
        if self.mask_mod is not None:
            mask = self.mask_mod(mask, b, s)
        h = self.attn(self.sa_norm(h), h, b, s, mask, input_pos)
        return self.mlp(self.mlp_norm(h), h)


class TPDecoder(nn.Module):
    """Forward returns the hidden states (or logits) of *this rank's* token rows, shaped ``[1, rows, ·]``;
    use :meth:`shard_rows` to cut labels the same way."""

    def __init__(self, model: TransformerDecoder, tp: TensorParallelContext, activation_checkpointing: bool = False, prepare_layer=None):
        super().__init__()
        self.tp = tp
        self.tok_embeddings, self.norm, self.output = model.tok_embeddings, model.norm, model.output
        layers = []
        for i, layer in enumerate(model.layers):
            inner = getattr(layer, "inner", layer)  # unwrap activation-checkpoint wrappers
            if not isinstance(inner, TransformerSelfAttentionLayer):
                raise NotImplementedError(f"tensor parallelism supports self-attention decoder layers, got {type(inner).__name__}")
            if prepare_layer is not None:  # the layer gets storage and values only now; its full weights are dropped right after slicing
                prepare_layer(inner, f"layers.{i}.")
            layers.append(TPLayer(inner, tp))
            _release_full_weights(inner)
        if prepare_layer is not None:
            for name in ("tok_embeddings", "norm", "output"):
                if isinstance(getattr(model, name), nn.Module):  # a tied output projection has no storage of its own
                    prepare_layer(getattr(model, name), f"{name}.")
        self.layers = nn.ModuleList(layers)
        self.max_seq_len = model.max_seq_len
        self.skip_output_layer = model.skip_output_layer
        self.activation_checkpointing = activation_checkpointing
        self._replicated = [p for m in (self.tok_embeddings, self.norm, self.output) for p in m.parameters()]
        for layer in self.layers:
            self._replicated += list(layer.sa_norm.parameters()) + list(layer.mlp_norm.parameters())
            if isinstance(layer.mlp, TPMoE):
                self._replicated += layer.mlp.replicated_parameters()
        seen = set()
        self._replicated = [p for p in self._replicated if not (id(p) in seen or seen.add(id(p)))]
        self._dp_group, self._dp_world = None, 1

    def set_data_parallel_group(self, group, size: int) -> None:
        """Under a dp × tp mesh: the process group of the ranks that hold the *same* shard (one per model replica) and its
        size.  Their gradients are summed in :meth:`sync_replicated_grads`."""
        self._dp_group, self._dp_world = group, int(size)

    def shard_rows(self, t: torch.Tensor) -> torch.Tensor:
        """``[b, s, …]`` → this rank's ``[1, b·s / tp, …]`` rows of the flattened token dimension."""
        flat = t.reshape(t.shape[0] * t.shape[1], *t.shape[2:])
        return _rows(flat, self.tp.rank, self.tp.world).unsqueeze(0)

    def forward(self, tokens: torch.Tensor, *, mask=None, input_pos: Optional[torch.Tensor] = None, **_: Any) -> torch.Tensor:
        b, s = tokens.shape
        if (b * s) % self.tp.world:
            raise ValueError(f"batch·seq ({b * s}) must be divisible by the tensor parallel size ({self.tp.world})")
        h = ops.embed_tokens(self.tok_embeddings, self.shard_rows(tokens)[0])
        for layer in self.layers:
            if self.activation_checkpointing and torch.is_grad_enabled():
                h = torch.utils.checkpoint.checkpoint(layer, h, b, s, mask, input_pos, use_reentrant=False)
            else:
                h = layer(h, b, s, mask, input_pos)
        h = self.norm(h).unsqueeze(0)
        return h if self.skip_output_layer else self.output(h).float()

    # inference ------------------------------------------------------------------------------
    def setup_caches(self, batch_size: int, dtype: torch.dtype, *, decoder_max_seq_len: Optional[int] = None, **_: Any) -> None:
        n = decoder_max_seq_len or self.max_seq_len
        for layer in self.layers:
            layer.attn.setup_cache(batch_size, dtype, n)

    def caches_are_setup(self) -> bool:
        return getattr(self.layers[0].attn, "kv_cache", None) is not None

    def caches_are_enabled(self) -> bool:
        return self.caches_are_setup()

    def reset_caches(self) -> None:
        for layer in self.layers:
            if getattr(layer.attn, "kv_cache", None) is not None:
                layer.attn.kv_cache.reset()

    @torch.no_grad()
    def forward_inference(self, tokens: Optional[torch.Tensor], *, mask=None, input_pos: Optional[torch.Tensor] = None, input_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Decoding-time forward: activations are replicated (any batch / sequence length, including one token), attention uses
        this rank's heads and KV cache, and the two row-parallel projections of every layer are followed by an all-reduce.
        ``input_embeds`` (``[b, s, d]``) replaces the embedding lookup (early-fusion models splice image embeddings in).
        Returns fp32 logits ``[b, s, vocab]``, identical on every rank."""
        h = ops.embed_tokens(self.tok_embeddings, tokens) if input_embeds is None else input_embeds
        for layer in self.layers:
            m = layer.mask_mod(mask, h.shape[0], h.shape[1]) if layer.mask_mod is not None else mask
            h = h + self.tp.all_reduce_(layer.attn.forward_replicated(layer.sa_norm(h), m, input_pos))
            h = h + self.tp.all_reduce_(layer.mlp.forward_replicated(layer.mlp_norm(h)))
        return self.output(self.norm(h)).float()

    def _sum_grads(self, grads, reduce_) -> None:
        # large tensors (embedding, output projection, projection shards) are reduced in place; only the many small ones (norm
        # scales) share a flat fp32 buffer — concatenating everything would stage gigabytes per step
        small = []
        for g in grads:
            if g.numel() >= (1 << 20) and g.is_cuda and g.is_contiguous():
                reduce_(g)
            else:
                small.append(g)
        if not small:
            return
        flat = torch.cat([g.reshape(-1).float() for g in small])
        reduce_(flat)
        off = 0
        for g in small:
            g.copy_(flat[off : off + g.numel()].view_as(g))
            off += g.numel()

    def sync_replicated_grads(self) -> None:
        """Sum the gradients of replicated parameters over the tensor-parallel group, then — under a dp × tp mesh — every
        gradient over the model replicas."""
        if self.tp.world > 1:
            self._sum_grads([p.grad for p in self._replicated if p.grad is not None], self.tp.all_reduce_)
        if self._dp_world > 1:
            group = self._dp_group

            def over_replicas(t: torch.Tensor) -> None:
                if t.device.type == "cpu" and t.dtype == torch.bfloat16:
                    f = t.float()
                    dist.all_reduce(f, group=group)
                    t.copy_(f)
                else:
                    dist.all_reduce(t, group=group)

            self._sum_grads([p.grad for p in self.parameters() if p.grad is not None], over_replicas)

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        """Checkpoint-layout state dict (every rank takes part in the gathers; all get the result)."""
        out: Dict[str, torch.Tensor] = {}
        for name, mod in (("tok_embeddings", self.tok_embeddings), ("norm", self.norm), ("output", self.output)):
            for k, v in mod.state_dict().items():
                out[f"{name}.{k}"] = v.detach()
        for i, layer in enumerate(self.layers):
            out.update(layer.attn.gather_full(f"layers.{i}.attn."))
            out.update(layer.mlp.gather_full(f"layers.{i}.mlp."))
            for nm in ("sa_norm", "mlp_norm"):
                for k, v in getattr(layer, nm).state_dict().items():
                    out[f"layers.{i}.{nm}.{k}"] = v.detach()
            for nm in ("q_norm", "k_norm"):
                norm = getattr(layer.attn, nm)
                if isinstance(norm, nn.Module):
                    for k, v in norm.state_dict().items():
                        out[f"layers.{i}.attn.{nm}.{k}"] = v.detach()
        return out


def _release_full_weights(inner: nn.Module) -> None:
    """Drop the unsharded projection weights of a converted layer (their slices were copied)."""
    projs = [inner.attn.q_proj, inner.attn.k_proj, inner.attn.v_proj, inner.attn.output_proj]
    mlp = inner.mlp
    if hasattr(mlp, "experts"):  # mixture of experts: the full expert stacks and the shared expert were copied in slices
        for name in ("gate_proj", "up_proj", "down_proj"):
            w = getattr(mlp.experts, name)
            w.data = torch.empty(0, dtype=w.dtype, device=w.device)
        mlp = mlp.shared_expert
    if mlp is not None:
        projs += [mlp.w1, mlp.w2, mlp.w3]
    for proj in projs:
        proj.weight.data = torch.empty(0, dtype=proj.weight.dtype, device=proj.weight.device)


def tensor_parallelize(model: TransformerDecoder, tp: TensorParallelContext, activation_checkpointing: bool = False, prepare_layer=None) -> TPDecoder:
    """Build the tensor-parallel model from a decoder that is either fully materialised (every rank: identical) or still on the
    meta device; in the second case ``prepare_layer(module, prefix)`` (e.g. :class:`training.LayerwisePreparer`) gives each
    layer storage and values right before it is sliced.  Full projection weights are released as each layer is converted, so
    at most one unsharded layer is alive at a time."""
    return TPDecoder(model, tp, activation_checkpointing, prepare_layer)
