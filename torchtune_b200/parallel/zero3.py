"""Fully sharded data parallelism (ZeRO-3): every parameter, gradient and optimizer moment is split over the ranks.

The reference wraps each decoder layer, the embedding and the output head in an FSDP2 unit: NCCL all-gather before the
unit's forward and again before its backward, NCCL reduce-scatter of the gradients, then ``scale_grads_`` and a
``torch.optim.AdamW`` step on the DTensor shards (torchtune/training/_distributed.py:612-714,
recipes/full_finetune_distributed.py:673-692, 1030-1050).  Here the same memory picture is built on peer memory:

* **layout** — the trainable parameters form one flat index space cut into buckets (one per decoder layer, one for what
  precedes the layers, one for what follows, :class:`~.dp.FlatLayout`); rank ``r`` owns slice ``r`` of every bucket and
  keeps it — with its AdamW moments — in a peer-visible *shard store*.  Nothing else of the model is resident.
* **gather** — a bucket becomes whole only while its layer runs: ``ttb_zero3_gather`` (``ops/csrc/comm.cu``) pulls the peers'
  slices over NVLink into a buffer from torch's allocator, one bucket ahead of the compute stream on a communication
  stream with a few dozen CTAs (NVLink-bound; they share the SMs with the GEMM kernels).  After the layer's forward the
  buffer's storage is released (the parameters are views of it, so they come back in place when it is gathered again for
  backward).
* **reduce-scatter → AdamW** — weight gradients are written by the GEMM epilogues into one of two peer-visible gradient
  slots (buckets alternate).  When a layer's backward is complete the owner of each slice pulls that slice from every
  rank's slot, sums in fp32 and applies AdamW to its shard *in the same kernel* (``ttb_dp_reduce_adamw_bcast`` without the
  broadcast): there is no reduced-gradient tensor, no separate scale pass and no optimizer step after backward.  With
  gradient clipping or gradient accumulation the kernel instead adds the reduced slice to an fp32 shard-sized buffer and the
  update follows once the global norm is known.
* **ordering** — readiness flags in peer memory (``ttb_dp_signal`` / bounded ``ttb_dp_wait``), three per bucket: gradients
  ready, slot consumed, shard updated.  No collective sits between the layers; the only NCCL call of a step is the scalar
  all-reduce of the token count (and of the squared norm when clipping).

Without CUDA (gloo) the same engine runs with ``all_gather`` / ``all_reduce`` in place of the kernels, so hooks, slot
rotation and the optimizer arithmetic are testable on CPU.
"""
from __future__ import annotations

import ctypes
import os
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn

from ..ops import reference as _ref
from .dp import FlatLayout, ShardedAdamW, _declare_dp
from .fabric import PeerBuffer


def _bf16_safe_all_reduce(t: torch.Tensor, group) -> None:
    if t.device.type == "cpu" and t.dtype == torch.bfloat16:
        f = t.float()
        dist.all_reduce(f, group=group)
        t.copy_(f)
    else:
        dist.all_reduce(t, group=group)


class ShardedParameters(FlatLayout):
    """Storage side of the engine: the shard store, the two gradient slots and one releasable full buffer per bucket."""

    def __init__(self, params: List[Tuple[str, nn.Parameter]], world: int, rank: int, device: torch.device, group=None, materialize=None):
        """``materialize(bucket) -> {name: parameter}`` (optional): for a model still on the meta device, gives the bucket's
        modules storage and values and returns their (new) parameter objects; buckets are then materialised one at a time and cut
        into shards at once, so the full model never exists on the device."""
        super().__init__(params, world)
        self.rank, self.device = rank, device
        esize = torch.empty(0, dtype=self.dtype).element_size()
        self.esize = esize
        self.store = PeerBuffer(self.shard * esize, device, group)
        self.shard_param = self.store.tensor(self.dtype, self.shard)
        self.flat_param = self.shard_param  # the optimizer asks this tensor for device / dtype
        self.max_bucket = max(size for _, size in self.buckets)
        self.grad_slots = [PeerBuffer(self.max_bucket * esize, device, group) for _ in range(2)]
        self.full: List[torch.Tensor] = []
        self.live: List[bool] = []
        self.gaps: List[List[Tuple[int, int]]] = []  # per bucket: (bucket-relative start, length) of padding between / after parameters
        self._registered: List[List[int]] = [[] for _ in self.buckets]
        index = {id(p): i for i, p in enumerate(self.params)}
        with torch.no_grad():
            for b, (start, size) in enumerate(self.buckets):
                if materialize is not None:
                    fresh = materialize(b)
                    for j, p in enumerate(self.bucket_params[b]):
                        i = index.pop(id(p))
                        new = fresh[self.names[i]]
                        self.params[i] = self.bucket_params[b][j] = new
                        index[id(new)] = i
                full = torch.zeros(size, dtype=self.dtype, device=device)
                slot = self.grad_slots[b % 2].tensor(self.dtype, self.max_bucket)
                cursor, gaps = 0, []
                for p in self.bucket_params[b]:
                    off = self.offsets[index[id(p)]] - start
                    if off > cursor:
                        gaps.append((cursor, off - cursor))
                    full[off : off + p.numel()].copy_(p.data.reshape(-1))
                    p.data = full[off : off + p.numel()].view(p.shape)
                    p._grad_buffer = slot[off : off + p.numel()].view(p.shape)
                    p._grad_written = False
                    cursor = off + p.numel()
                if size > cursor:
                    gaps.append((cursor, size - cursor))
                begin, count, soff = self.owned(b, rank)
                self.shard_param[soff : soff + count].copy_(full[begin - start : begin - start + count])
                self.full.append(full)
                self.live.append(True)
                self.gaps.append(gaps)
                self.release(b)

    # bucket storage ------------------------------------------------------------------------
    def allocate(self, b: int) -> None:
        if self.live[b]:
            return
        full = self.full[b]
        full.untyped_storage().resize_(full.numel() * self.esize)
        self.live[b] = True
        if self.device.type == "cuda":
            from ..ops import _cuda

            for p in self.bucket_params[b]:
                _cuda.register_grad_window(p)
                self._registered[b].append(p.data_ptr())

    def release(self, b: int) -> None:
        if not self.live[b]:
            return
        if self.device.type == "cuda" and self._registered[b]:
            from ..ops import _cuda

            for ptr in self._registered[b]:
                _cuda.unregister_grad_window(ptr)
            self._registered[b] = []
        self.full[b].untyped_storage().resize_(0)
        self.live[b] = False

    def grad_view(self, b: int) -> torch.Tensor:
        return self.grad_slots[b % 2].tensor(self.dtype, self.buckets[b][1])

    def zero_gaps(self, b: int) -> None:
        """The padding inside a bucket's gradient slot still holds another bucket's values: clear it so that norms and moments
        of the padding stay zero."""
        g = self.grad_view(b)
        for start, n in self.gaps[b]:
            g[start : start + n].zero_()

    def close(self) -> None:
        self.store.close()
        for s in self.grad_slots:
            s.close()


class Zero3AdamW(ShardedAdamW):
    """AdamW on this rank's parameter shards; the reduce → update kernel is launched per bucket by the engine as soon as the
    bucket's gradients are final.  State and checkpoint form are those of :class:`~.dp.ShardedAdamW`."""

    def __init__(self, sp: ShardedParameters, rank: int, world: int, **kw: Any):
        super().__init__(sp, rank, world, **kw)
        self.reduced: set = set()  # buckets whose reduced gradient sits in the fp32 buffer (deferred update)

    def ensure_gsum(self) -> None:
        if self._gsum is None:
            self._gsum = torch.zeros(self.flat.shard, dtype=torch.float32, device=self.flat.shard_param.device)

    def begin_step(self, grad_scale, max_grad_norm) -> None:
        super().begin_step(grad_scale, max_grad_norm)
        sp = self.flat
        if sp.shard_param.is_cuda:
            from ..ops._lib import lib

            grid = lib().ttb_dp_grid()
            if self._partials is None:
                self._partials = torch.zeros(len(sp.buckets) * grid, dtype=torch.float32, device=sp.shard_param.device)
            self._open["grid"] = grid

    def _launch(self, bucket: int, mode: int, st: Dict[str, Any], sdev, shost, wait=None, grid_ctas: int = 0, accumulate: bool = False) -> None:
        from ..ops._lib import check, err_word, lib, stream_ptr

        L = lib()
        _declare_dp(L)
        sp, g = self.flat, self.param_groups[0]
        _, piece, soff = sp.owned(bucket, self.rank)
        begin = self.rank * piece  # bucket-relative start of this rank's slice
        grads = sp.grad_slots[bucket % 2].pointer_array()
        # the kernel addresses parameters as base[rank] + begin + i; only this rank's entry is used (bcast = 0)
        params = (ctypes.c_void_p * self.world)(*[sp.store.local_ptr + sp.esize * (soff - begin)] * self.world)
        esz = self.exp_avg.element_size()
        b1, b2 = g["betas"]
        gsum = None if mode == 0 else self._gsum.data_ptr() + 4 * soff
        grid = st.get("grid") or L.ttb_dp_grid()
        partials = None if mode != 1 else self._partials.data_ptr() + 4 * bucket * grid
        check(
            L.ttb_dp_reduce_adamw_bcast(grads, params, self.world, self.rank, begin, piece, self.exp_avg.data_ptr() + esz * soff, self.exp_avg_sq.data_ptr() + esz * soff,
                                        gsum, partials, None if sdev is None else sdev.data_ptr(), shost, float(g["lr"]), b1, b2, g["eps"], g["weight_decay"],
                                        st["inv_bc1"], st["inv_sqrt_bc2"], mode, None if wait is None else wait[0], 0 if wait is None else wait[1], 0 if wait is None else wait[2],
                                        err_word(sp.device).data_ptr(), int(grid_ctas), 0, int(accumulate), stream_ptr()),
            "zero3 reduce + adamw",
        )

    # host statements of the same three kernels ------------------------------------------------
    def host_reduce(self, bucket: int, group, fused: bool, st: Dict[str, Any]) -> None:
        sp, g = self.flat, self.param_groups[0]
        _, piece, soff = sp.owned(bucket, self.rank)
        summed = sp.grad_view(bucket).float()
        if self.world > 1:
            dist.all_reduce(summed, group=group)
        mine = summed[self.rank * piece : (self.rank + 1) * piece]
        if fused:
            scale = float(st["scale_dev"].item()) if st["scale_dev"] is not None else st["scale_host"]
            self._host_adamw(soff, piece, mine, scale)
            return
        self.ensure_gsum()
        if bucket in self.reduced:
            self._gsum[soff : soff + piece] += mine
        else:
            self._gsum[soff : soff + piece] = mine
        self.reduced.add(bucket)

    def _host_adamw(self, soff: int, piece: int, grad: torch.Tensor, scale: float) -> None:
        g = self.param_groups[0]
        b1, b2 = g["betas"]
        sl = slice(soff, soff + piece)
        new = self.flat.shard_param[sl].clone()
        m, v = self.exp_avg[sl].clone(), self.exp_avg_sq[sl].clone()
        _ref.adamw_step(new, grad, m, v, self.step_count, float(g["lr"]), b1, b2, g["eps"], g["weight_decay"], scale)
        self.flat.shard_param[sl] = new
        self.exp_avg[sl], self.exp_avg_sq[sl] = m, v

    def local_sumsq(self) -> torch.Tensor:
        if not self.flat.shard_param.is_cuda:
            return self._gsum.pow(2).sum()
        return self._partials.sum()

    def finish(self, total_sumsq: Optional[torch.Tensor]) -> None:
        """Deferred update of every bucket from the fp32 reduced gradient (after clipping / gradient accumulation)."""
        st, sp = self._open, self.flat
        self.last_grad_norm = None
        try:
            dev = sp.shard_param.device
            s = st["scale_dev"].to(dev) if st["scale_dev"] is not None else torch.tensor([st["scale_host"]], dtype=torch.float32, device=dev)
            coef = s
            if st["clip"] is not None:
                norm = total_sumsq.to(torch.float32).sqrt() * s
                self.last_grad_norm = norm.reshape(())
                coef = (torch.clamp(float(st["clip"]) / (norm + 1e-6), max=1.0) * s).reshape(1).float()
            for b in sorted(self.reduced):
                if sp.shard_param.is_cuda:
                    self._launch(b, 2, st, coef.reshape(1).float(), 1.0)
                else:
                    _, piece, soff = sp.owned(b, self.rank)
                    self._host_adamw(soff, piece, self._gsum[soff : soff + piece], float(coef.item()))
            self.reduced.clear()
            if self._partials is not None:
                self._partials.zero_()
        finally:
            self._open = None


class Zero3Engine:
    """Hooks, streams and flags around :class:`ShardedParameters`; the recipe-facing surface matches
    :class:`~.dp.DataParallelEngine` (``prepare``, ``build_optimizer``, ``arm_backward_overlap``, ``optimizer_step`` …)."""

    RDY, CONS, UPD = 0, 1, 2  # flag kinds; bucket b uses slots 3·b + kind

    def __init__(self, device: torch.device, group=None, replica_group=None):
        """``group``: the ranks the parameters are sharded over (``None`` = every rank).  ``replica_group`` (hybrid sharding,
        ``data_parallel_replicate_dim`` > 1): the ranks that hold the *same* shard in the other shard groups; their reduced
        gradients are summed with one all-reduce of the fp32 shard per step before the update (so the update is never fused
        into backward in this mode)."""
        self.device, self.group, self.replica_group = device, group, replica_group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.replicas = dist.get_world_size(replica_group) if (replica_group is not None and dist.is_initialized()) else 1
        self.global_rank = dist.get_rank() if dist.is_initialized() else 0
        self.cuda = device.type == "cuda"
        self.sp: Optional[ShardedParameters] = None
        self.optimizer: Optional[Zero3AdamW] = None
        self._armed = False
        self._comm = None
        self._flags: Optional[PeerBuffer] = None
        self._token = torch.zeros(1, device=device if self.cuda else "cpu")
        # CTAs of the kernels that run beside the layers' GEMMs; 0 = full grid.  The bytes a rank moves per bucket shrink with the
        # world size (1/world of the gradients and moments, NVLink-bound pulls), so fewer CTAs keep up on more ranks and leave
        # more of the SMs' issue slots and of the HBM to the GEMMs.
        self.comm_ctas = int(os.environ.get("TTB_ZERO3_CTAS", "0")) or max(48, 592 // max(self.world, 1))

    dp_size = property(lambda self: self.world * self.replicas)  # every rank reads its own batches
    dp_rank = property(lambda self: self.global_rank if self.replicas > 1 else self.rank)
    non_data_parallel_size = 1
    min_seq_len_divisor = 1

    # ------------------------------------------------------------------ setup
    def prepare(self, model: nn.Module, prepare_layer=None) -> nn.Module:
        """Shard ``model`` in place.  ``prepare_layer(module, prefix)`` (e.g. :class:`training.LayerwisePreparer`): the model is still
        on the meta device and every bucket's modules get storage and values right before they are cut into shards."""
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        materialize = None
        if prepare_layer is not None:
            layout = FlatLayout(named, self.world)

            def materialize(b: int) -> Dict[str, nn.Parameter]:
                key = layout.bucket_keys[b]
                if key is not None:
                    prepare_layer(model.get_submodule(key), key + ".")
                else:  # direct owner modules of the parameters before / after the layers
                    owners = {n.rsplit(".", 1)[0] if "." in n else "" for n, p in named if any(p is q for q in layout.bucket_params[b])}
                    for path in sorted(owners):
                        prepare_layer(model.get_submodule(path) if path else model, path + "." if path else "")
                return dict(model.named_parameters())

        self.sp = sp = ShardedParameters(named, self.world, self.rank, self.device, self.group, materialize)
        if prepare_layer is not None:
            for mod in model.modules():  # buffers outside every bucket's modules (e.g. a shared RoPE table)
                meta = [k for k, buf in mod._buffers.items() if buf is not None and buf.is_meta]
                for k in meta:
                    mod._buffers[k] = torch.empty_like(mod._buffers[k], device=self.device)
                if meta and hasattr(mod, "rope_init"):
                    with self.device:
                        mod.rope_init()
            left = [n for n, p in model.named_parameters() if p.is_meta]
            if left:
                raise NotImplementedError(f"frozen parameters of a meta-device model are not materialised by the sharded-parameter engine: {left[:4]}")
        nb = len(sp.buckets)
        self.nb = nb
        self._gather_event: List[Any] = [None] * nb
        self._reduce_event: List[Any] = [None] * nb
        self._slot_user: List[Optional[int]] = [None, None]  # bucket whose gradients occupy each slot
        self._micro = [0] * nb  # hand-overs of each bucket so far (epoch of its RDY / CONS flags)
        self._updates = [0] * nb  # optimizer updates of each bucket so far (epoch of its UPD flag)
        self._pending = [False] * nb  # gradient slot acquired, bucket not handed over yet
        self._handed = [False] * nb  # handed over in the running backward pass
        self._layer_buckets = [b for b, k in enumerate(sp.bucket_keys) if k is not None]
        # an embedding table is not read by its own backward: buckets made only of embeddings are not gathered again
        emb = {id(p) for m in model.modules() if isinstance(m, nn.Embedding) for p in m.parameters(recurse=False)}
        self._regather = [not all(id(p) in emb for p in ps) for ps in sp.bucket_params]
        if self.cuda:
            from ..ops import _cuda
            from ..ops._lib import lib

            L = lib()
            _declare_dp(L)
            if 3 * nb >= L.ttb_dp_max_buckets():
                raise ValueError(f"{nb} parameter buckets exceed the flag array of the sharded-parameter engine")
            _cuda.enable_direct_wgrad(True)
            self._comm = torch.cuda.Stream(device=self.device)  # reduce-scatter → AdamW kernels
            self._gstream = torch.cuda.Stream(device=self.device)  # parameter gathers (never queued behind a reduction)
            self._flags = PeerBuffer(self.world * L.ttb_dp_max_buckets() * 4, self.device, self.group)
        self._install_hooks(model)
        self._model = model
        return model

    def _install_hooks(self, model: nn.Module) -> None:
        """Decoder layers get module hooks.  What precedes the layers (the embedding table, which the decoder reads without
        calling the module) is gathered when the model's forward starts and let go when the first layer starts; what follows
        them (final norm, output head — read by the fused loss after the model has returned) is gathered when the last layer
        ends and let go once its gradients are handed over."""
        sp = self.sp
        if not self._layer_buckets:
            raise NotImplementedError("sharded parameters need a model with decoder layers (module paths ending in layers.<n>)")
        first, last = self._layer_buckets[0], self._layer_buckets[-1]
        self._last_layer = last
        self._head = list(range(0, first))
        self._tail = list(range(last + 1, self.nb))
        for b in self._layer_buckets:
            mod = model.get_submodule(sp.bucket_keys[b])
            mod.register_forward_pre_hook(lambda m, args, b=b: self._pre_forward(b, args[0] if args else None))
            mod.register_forward_hook(lambda m, args, out, b=b: self._post_forward(b, out))
        model.register_forward_pre_hook(lambda m, args: self._model_pre_forward())
        model.register_forward_hook(lambda m, args, out: self._after_model_forward())

    @staticmethod
    def _first_tensor(x: Any) -> Optional[torch.Tensor]:
        if torch.is_tensor(x):
            return x
        if isinstance(x, (tuple, list)) and x and torch.is_tensor(x[0]):
            return x[0]
        return None

    def _watch(self, x: Any, fn) -> None:
        t = self._first_tensor(x)
        if t is not None and t.requires_grad and torch.is_grad_enabled():
            t.register_hook(lambda g: fn())

    # ------------------------------------------------------------------ forward
    def _model_pre_forward(self) -> None:
        for t in self._tail:  # left whole by an earlier gradient-free pass
            if self.sp.live[t] and not self._pending[t]:
                self._release(t)
        for b in self._head:
            if self._pending[b]:
                self._after_backward(b)  # gradients of an earlier micro-batch that no hook handed over
            self._handed[b] = False
            self._ensure(b)
        self._prefetch(self._layer_buckets[0])

    def _pre_forward(self, b: int, x: Any) -> None:
        if self._pending[b]:
            self._after_backward(b)
        self._handed[b] = False
        self._ensure(b)
        grad = torch.is_grad_enabled()
        if b == self._layer_buckets[0]:
            for hb in self._head:
                if grad and x is not None:
                    self._watch(x, lambda hb=hb: self._before_backward(hb))
                self._release(hb)
        nxt = b + 1
        if nxt < self.nb and not self.sp.live[nxt]:
            self._prefetch(nxt)
        if grad and x is not None:
            self._watch(x, lambda: self._after_backward(b))

    def _post_forward(self, b: int, out: Any) -> None:
        grad = torch.is_grad_enabled()
        if grad:
            self._watch(out, lambda: self._before_backward(b))
        if b != self._last_layer:
            self._release(b)
            return
        if not grad:
            self._release(b)  # (with gradients the last layer's parameters are needed again at once by backward)
        for t in self._tail:
            if self._pending[t]:
                self._after_backward(t)
            self._handed[t] = False
            self._ensure(t)
            if grad:
                self._acquire_slot(t)  # the fused loss writes the output head's gradient during forward
                # the gradient of the last layer's output is complete once everything behind the layers has run backward
                self._watch(out, lambda t=t: self._after_backward(t))

    def _after_model_forward(self) -> None:
        # Without gradients nothing will ask for the layers again.  What follows them stays whole (a fused loss reads the output
        # projection after the model has returned) until the next forward pass starts.
        if not torch.is_grad_enabled():
            for b in self._head + self._layer_buckets:
                self._release(b)

    # ------------------------------------------------------------------ gather
    def _release(self, b: int) -> None:
        """Give the bucket's storage back.  A gather still in flight on the communication stream is waited for first: the
        allocator hands the block to the compute stream's next request at once."""
        ev = self._gather_event[b]
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
            self._gather_event[b] = None
        self.sp.release(b)

    def _ensure(self, b: int) -> None:
        """Bucket ``b`` whole and visible to the compute stream."""
        if not self.sp.live[b]:
            self._issue_gather(b)
        ev = self._gather_event[b]
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
            self._gather_event[b] = None

    def _prefetch(self, b: int) -> None:
        if 0 <= b < self.nb and not self.sp.live[b]:
            self._issue_gather(b)

    def _issue_gather(self, b: int) -> None:
        sp = self.sp
        sp.allocate(b)
        _, piece, soff = sp.owned(b, self.rank)
        full = sp.full[b]
        if not self.cuda:
            mine = sp.shard_param[soff : soff + piece]
            if self.world > 1:
                parts = [torch.empty(piece, dtype=torch.float32) for _ in range(self.world)]
                dist.all_gather(parts, mine.float().contiguous(), group=self.group)
                full.copy_(torch.cat(parts).to(full.dtype))
            else:
                full.copy_(mine)
            return
        from ..ops._lib import check, err_word, lib, stream_ptr

        main = torch.cuda.current_stream(self.device)
        self._gstream.wait_stream(main)  # the buffer may be a block the compute stream has just freed; also orders behind updates issued there
        if self._reduce_event[b] is not None:
            self._gstream.wait_event(self._reduce_event[b])  # this rank's own update of the bucket's shard
        with torch.cuda.stream(self._gstream):
            ptrs = (ctypes.c_void_p * self.world)(*[p + sp.esize * soff for p in sp.store.peer_ptrs])
            wait = self._flags.local_ptr if (self.world > 1 and self._updates[b] > 0) else None
            check(lib().ttb_zero3_gather(ptrs, self.world, self.rank, piece, full.data_ptr(), wait, 3 * b + self.UPD, self._updates[b],
                                         err_word(self.device).data_ptr(), self.comm_ctas if self.world > 1 else 0, stream_ptr()), "zero3 gather")
            ev = torch.cuda.Event()
            ev.record(self._gstream)
        self._gather_event[b] = ev

    # ------------------------------------------------------------------ backward
    def _acquire_slot(self, b: int) -> None:
        """Make the gradient slot of bucket ``b`` writable: its previous user's slice must have been pulled by every rank."""
        s = b % 2
        prev = self._slot_user[s]
        if prev is not None and prev != b and self.cuda:
            if self._pending[prev]:
                self._after_backward(prev)
            ev = self._reduce_event[prev]
            main = torch.cuda.current_stream(self.device)
            if ev is not None:
                main.wait_event(ev)
            if self.world > 1 and self._micro[prev] > 0:
                from ..ops._lib import check, err_word, lib, stream_ptr

                check(lib().ttb_dp_wait(self._flags.local_ptr, self.world, self.rank, 3 * prev + self.CONS, self._micro[prev], err_word(self.device).data_ptr(), stream_ptr()), "zero3 slot wait")
        elif prev is not None and prev != b and self._pending[prev]:
            self._after_backward(prev)
        self._slot_user[s] = b
        self.sp.zero_gaps(b)
        self._pending[b] = True

    def _before_backward(self, b: int) -> None:
        if self._handed[b]:
            return
        if self._regather[b]:
            self._ensure(b)
            if self._layer_buckets and b > self._layer_buckets[0]:
                self._prefetch(b - 1)
        if not self._pending[b]:
            self._acquire_slot(b)

    def _after_backward(self, b: int) -> None:
        """Gradients of bucket ``b`` are final on this rank: hand them to the owners (reduce → AdamW, or reduce into the fp32 buffer)."""
        if self._handed[b] and not self._pending[b]:
            return
        if not self._pending[b]:
            self._acquire_slot(b)  # nothing wrote a gradient (frozen path): the slot still has to be defined
        sp, opt = self.sp, self.optimizer
        sp.collect_autograd_grads(b)
        for p in sp.bucket_params[b]:
            p._grad_written = False  # the slot's content is consumed by this hand-over: the next backward pass starts afresh
        self._pending[b] = False
        self._handed[b] = True
        self._micro[b] += 1
        fused = self._armed and opt._open is not None and opt._open["clip"] is None
        if opt._open is None:
            opt.begin_step(1.0, None)  # deferred update: scale and clipping arrive with optimizer_step
            opt._open["deferred"] = True
        st = opt._open
        if not self.cuda:
            opt.host_reduce(b, self.group, fused, st)
            if fused:
                self._updates[b] += 1
            self._release(b)
            return
        from ..ops import _cuda
        from ..ops._lib import check, lib, stream_ptr

        L = lib()
        main = torch.cuda.current_stream(self.device)
        self._comm.wait_stream(main)
        if _cuda._wgrad_stream is not None:
            self._comm.wait_stream(_cuda._wgrad_stream)
        with torch.cuda.stream(self._comm):
            flags = self._flags.pointer_array()
            wait = None
            if self.world > 1:
                check(L.ttb_dp_signal(flags, self.world, self.rank, 3 * b + self.RDY, self._micro[b], stream_ptr()), "zero3 signal")
                wait = (self._flags.local_ptr, 3 * b + self.RDY, self._micro[b])
            ctas = self.comm_ctas if self.world > 1 else 0
            if fused:
                opt._launch(b, 0, st, st["scale_dev"], st["scale_host"], wait=wait, grid_ctas=ctas)
                self._updates[b] += 1
            else:
                opt.ensure_gsum()
                opt._launch(b, 1, st, None, 1.0, wait=wait, grid_ctas=ctas, accumulate=b in opt.reduced)
                opt.reduced.add(b)
            if self.world > 1:
                check(L.ttb_dp_signal(flags, self.world, self.rank, 3 * b + self.CONS, self._micro[b], stream_ptr()), "zero3 signal")
                if fused:
                    check(L.ttb_dp_signal(flags, self.world, self.rank, 3 * b + self.UPD, self._updates[b], stream_ptr()), "zero3 signal")
            ev = torch.cuda.Event()
            ev.record(self._comm)
        self._reduce_event[b] = ev
        self._release(b)

    # ------------------------------------------------------------------ step protocol (same surface as DataParallelEngine)
    def build_optimizer(self, model: nn.Module, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2, **_: Any) -> Zero3AdamW:
        if self.sp is None:
            raise RuntimeError("call prepare(model) first")
        self.optimizer = Zero3AdamW(self.sp, self.rank, self.world, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, group=self.group)
        return self.optimizer

    def wants_backward_overlap(self, optimizer) -> bool:
        return self.replicas == 1 and optimizer is not None and optimizer is self.optimizer and not self._armed and optimizer._open is None

    def arm_backward_overlap(self, optimizer, grad_scale, clip_grad_norm: Optional[float] = None) -> bool:
        """Call between forward and ``backward()`` of the step's only (or last) micro-batch with the final gradient scale: every
        bucket is then reduced *and updated* as soon as its layer's backward is complete."""
        if not self.wants_backward_overlap(optimizer):
            return False
        optimizer.begin_step(grad_scale, clip_grad_norm)
        self._armed = True
        return True

    def all_reduce_sum_(self, *tensors: torch.Tensor) -> None:
        """Sum over every data-parallel rank (all shard groups)."""
        if self.world * self.replicas == 1:
            return
        everyone = self.group if self.replicas == 1 else None
        if len(tensors) == 1:
            dist.all_reduce(tensors[0], group=everyone)
            return
        packed = torch.stack([t.reshape(()).to(torch.float32) for t in tensors])
        dist.all_reduce(packed, group=everyone)
        for t, v in zip(tensors, packed):
            t.copy_(v)

    def barrier(self) -> None:
        if self.world * self.replicas > 1:
            dist.all_reduce(self._token, group=self.group if self.replicas == 1 else None)

    def optimizer_step(self, model: nn.Module, optimizer: Zero3AdamW, grad_scale, clip_grad_norm: Optional[float] = None):
        if optimizer is not self.optimizer:
            raise RuntimeError("optimizer_step was called with another optimizer than the one this engine built")
        for b in range(self.nb - 1, -1, -1):  # whatever no hook handed over (the embedding; frozen inputs)
            if self._pending[b] or not self._handed[b]:
                self._after_backward(b)
        st = optimizer._open
        deferred = st is not None and (st.get("deferred") or st["clip"] is not None)
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self._comm)
        if deferred:
            if st.get("deferred"):  # opened by a hand-over without scale: take the step's real scale and clipping now
                if isinstance(grad_scale, torch.Tensor):
                    st["scale_dev"] = grad_scale.detach().to(torch.float32).reshape(1)
                else:
                    st["scale_host"] = float(grad_scale)
                st["clip"] = clip_grad_norm
            if self.replicas > 1:  # hybrid sharding: the same slices of the other shard groups
                dist.all_reduce(optimizer._gsum, group=self.replica_group)
            total = None
            if st["clip"] is not None:
                total = optimizer._gsum.pow(2).sum() if self.replicas > 1 else optimizer.local_sumsq()
                if self.world > 1:
                    dist.all_reduce(total, group=self.group)
            updated = sorted(optimizer.reduced)
            optimizer.finish(total)
            for b in updated:
                self._updates[b] += 1
                if self.cuda and self.world > 1:
                    from ..ops._lib import check, lib, stream_ptr

                    check(lib().ttb_dp_signal(self._flags.pointer_array(), self.world, self.rank, 3 * b + self.UPD, self._updates[b], stream_ptr()), "zero3 signal")
        else:
            optimizer._open = None
            optimizer.last_grad_norm = None
        self._armed = False
        self._handed = [False] * self.nb
        optimizer.zero_grad()
        return optimizer.last_grad_norm

    # ------------------------------------------------------------------ checkpoints
    def full_state_dict(self, model: nn.Module, to_cpu: bool = True) -> Dict[str, torch.Tensor]:
        """Checkpoint-layout state dict (collective: every rank gathers every bucket); buffers are taken as they are."""
        sp = self.sp
        names = {id(p): n for n, p in model.named_parameters()}
        out: Dict[str, torch.Tensor] = {}
        for b in range(self.nb):
            was_live = sp.live[b]
            self._ensure(b)
            if self.cuda:
                torch.cuda.current_stream(self.device).synchronize()
            for p in sp.bucket_params[b]:
                out[names[id(p)]] = p.detach().cpu().clone() if to_cpu else p.detach().clone()
            if not was_live:
                self._release(b)
        for k, v in model.state_dict().items():
            if k not in out and v.untyped_storage().size() > 0:
                out[k] = v.detach().cpu() if to_cpu else v.detach()
        return out

    def shutdown(self) -> None:
        if self.sp is not None:
            if self.cuda:
                torch.cuda.synchronize(self.device)
            self.barrier()
            if self._flags is not None:
                self._flags.close()
                self._flags = None
            self.sp.close()
            self.sp = None
