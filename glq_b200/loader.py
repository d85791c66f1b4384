"""Loader-side glue: what a serving framework calls between "here is a layer and its shapes" and "run it".

Mirrors the method names and argument meaning of the reference's vLLM plugin (``GLQLinearMethod`` in
glq_vllm/linear_method.py: ``create_weights`` :776, the weight loader :187-231, ``process_weights_after_loading``
:1031, ``apply`` :1466) without importing vLLM, so the same object serves vLLM (subclass ``LinearMethodBase`` and
delegate), another engine, or a plain script.  Differences that the B200 library makes possible:

* activations may be bf16 or fp16 (the reference casts to fp16);
* merged layers (q/k/v, gate/up) run as ONE launch over their shards (``fused_linear_trellis_3inst_shards``)
  instead of one op per shard plus a concatenation;
* everything that needs the host — scalar buffers, block decompositions, the packed codebook, decode plans and
  the workspace — is resolved once in ``process_weights_after_loading``; ``apply`` never synchronises;
* tensor parallelism: a checkpoint quantized per rank (every rank's shard its own GLQ layer, stored under
  ``<layer>.tp<G>.<r>.<buffer>``) is loaded shard-wise, row-parallel layers are summed over the ranks inside the
  decode kernel (``glq_b200.comm``); a checkpoint without such shards is replicated on every rank, which is all the
  reference does (its loader copies full tensors to every rank).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from . import ops
from .checkpoint import CheckpointError, QuantizeConfig, trellis_rates, validate_layer
from .plan import block_decompose

_E8_CODES = ("Qidxs", "Qidxs2", "Qidxs3", "Qidxs4")
_E8_SCALES = ("inv_resid_scale", "inv_resid_scale2", "inv_resid_scale3")


def tp_buffer_key(prefix: str, buffer: str, world: int, rank: int) -> str:
    """Name of a per-rank buffer in a checkpoint quantized for ``world`` tensor-parallel ranks."""
    return f"{prefix}.tp{world}.{rank}.{buffer}"


class ShardBuffers:
    """Per-shard storage of one buffer of a merged layer (the role of the reference's ``GLQShardedParameter``):
    shard i is whatever tensor the checkpoint holds for it, or empty when it was never loaded."""

    def __init__(self, n_shards: int, dtype: torch.dtype):
        self.dtype = dtype
        self.shards: List[torch.Tensor] = [torch.empty(0, dtype=dtype) for _ in range(n_shards)]

    def load(self, shard: int, t: torch.Tensor) -> None:
        if t.dtype != self.dtype:
            raise CheckpointError(f"shard {shard}: buffer is {t.dtype}, expected {self.dtype}")
        self.shards[shard] = t.detach()

    def get_shard(self, i: int) -> torch.Tensor:
        return self.shards[i]

    def to(self, device) -> None:
        self.shards = [s.to(device) for s in self.shards]


_SHARD_IDS = {"q": 0, "k": 1, "v": 2, 0: 0, 1: 1, 2: 2}


class LinearMethod:
    """One instance per (config, rate).  ``comm``: a ``glq_b200.comm.Comm`` when the model runs tensor parallel."""

    def __init__(self, config: QuantizeConfig, bpw: Optional[int] = None, codebook=None, codebook2=None, comm=None):
        self.config = config
        self.bpw = int(bpw if bpw is not None else config.bpw)
        self.codebook, self.codebook2 = codebook, codebook2      # E8: fp16 (65536, 8) and (256, 8) tables
        self.comm = comm
        if config.codebook == "e8_shell" and codebook is None:
            raise CheckpointError("E8 shell layers need the shared codebook table")

    # ---- create_weights -----------------------------------------------------------------------------------
    def create_weights(self, layer, input_size_per_partition: int, output_partition_sizes: Sequence[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra) -> None:
        """Attach empty GLQ buffers of the checkpoint's shapes to ``layer``.  More than one output partition = a
        merged layer whose parts were quantized separately (q/k/v, gate/up): per-shard buffers."""
        if params_dtype not in (torch.float16, torch.bfloat16, torch.float32):
            raise CheckpointError(f"activations of dtype {params_dtype} are not served")
        sizes = [int(s) for s in output_partition_sizes]
        trellis = self.config.codebook == "trellis"
        n = int(input_size_per_partition)
        if trellis:
            for m in sizes:
                if m % 32 or n % 32:
                    raise CheckpointError(f"trellis layers are stored unpadded in 32 x 32 groups: shard {m} x {n} does not "
                                          f"fit (reduce the tensor-parallel size)")
        elif n % 8:
            raise CheckpointError(f"E8 layers need an input width that is a multiple of 8, got {n}")
        layer.glq_in_features, layer.glq_shard_sizes = n, sizes
        layer.glq_is_fused = len(sizes) > 1
        layer.glq_is_trellis = trellis
        layer.glq_params_dtype = params_dtype
        layer.glq_row_parallel = bool(extra.get("row_parallel", False))
        ns = len(sizes)
        if trellis:
            names = {"trellis_packed": torch.int16, "trellis_packed2": torch.int16, "inv_resid_scale2": torch.float32}
        else:
            names = {k: torch.int16 for k in _E8_CODES}
            names.update({k: torch.float32 for k in _E8_SCALES})
        names.update({"SU": torch.float16, "SV": torch.float16, "Wscale": torch.float32})
        layer.glq_buffers = {k: ShardBuffers(ns, dt) for k, dt in names.items()}
        layer.glq_ready = False

    # ---- weight loader ------------------------------------------------------------------------------------
    def load_weight(self, layer, buffer: str, loaded: torch.Tensor, shard_id=None) -> None:
        """Place one checkpoint tensor.  ``shard_id``: position in a merged layer (0.. or 'q'/'k'/'v'); None for a
        layer that is stored whole."""
        if buffer == "tlut":
            if loaded.numel():
                raise CheckpointError("HYB (tlut) trellis layers are not served")
            return
        bufs: Dict[str, ShardBuffers] = layer.glq_buffers
        if buffer not in bufs:
            raise CheckpointError(f"buffer {buffer!r} does not belong to a {self.config.codebook} layer")
        i = 0 if shard_id is None else _SHARD_IDS.get(shard_id, shard_id)
        if not isinstance(i, int) or not 0 <= i < len(layer.glq_shard_sizes):
            raise CheckpointError(f"shard id {shard_id!r} outside a layer of {len(layer.glq_shard_sizes)} shards")
        bufs[buffer].load(i, loaded)
        layer.glq_ready = False

    def load_from(self, layer, tensors, prefixes: Sequence[str]) -> None:
        """Load a layer from a mapping of checkpoint tensors (or a ``checkpoint.Checkpoint``): one prefix per shard.
        Under tensor parallelism the rank's own ``.tp<G>.<r>.`` buffers are taken when the checkpoint has them."""
        get = tensors.tensor if hasattr(tensors, "tensor") else tensors.__getitem__
        has = (lambda k: k in tensors._where) if hasattr(tensors, "_where") else tensors.__contains__
        if len(prefixes) != len(layer.glq_shard_sizes):
            raise CheckpointError(f"{len(prefixes)} checkpoint layers for {len(layer.glq_shard_sizes)} shards")
        world = self.comm.world if self.comm is not None else 1
        rank = self.comm.rank if self.comm is not None else 0
        layer.glq_tp_sharded = False
        for i, prefix in enumerate(prefixes):
            for name in layer.glq_buffers:
                key = f"{prefix}.{name}"
                if world > 1 and has(tp_buffer_key(prefix, name, world, rank)):
                    key = tp_buffer_key(prefix, name, world, rank)
                    layer.glq_tp_sharded = True
                if has(key):
                    self.load_weight(layer, name, get(key), i if layer.glq_is_fused else None)

    # ---- process_weights_after_loading ----------------------------------------------------------------------
    def process_weights_after_loading(self, layer, device=None) -> None:
        """Move the buffers to the device, validate every shard, hoist the scalars, and warm the decode plan of one
        token (which also sizes the shared workspace), so that the first ``apply`` allocates nothing but its output."""
        device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        bufs: Dict[str, ShardBuffers] = layer.glq_buffers
        for b in bufs.values():
            b.to(device)
        meta = []
        for i, m in enumerate(layer.glq_shard_sizes):
            shard = {k: b.get_shard(i) for k, b in bufs.items() if b.get_shard(i).numel()}
            info = validate_layer(shard, self.config.codebook, f"shard {i}")
            n_in = layer.glq_in_features
            if layer.glq_is_trellis:
                if (info.m_pad, info.n_pad) != (m, n_in):
                    raise CheckpointError(f"shard {i}: checkpoint holds {info.m_pad} x {info.n_pad}, the layer is {m} x {n_in}")
            elif info.m_pad < m or info.n_pad < n_in:
                raise CheckpointError(f"shard {i}: checkpoint holds {info.m_pad} x {info.n_pad}, smaller than the layer {m} x {n_in}")
            d = {"m": m, "m_pad": info.m_pad, "n_pad": info.n_pad, "n_stages": info.n_stages,
                 "wscale": float(shard["Wscale"].item()), "block_diagonal": info.block_diagonal,
                 "blocks_m": block_decompose(info.m_pad) if info.block_diagonal else [info.m_pad],
                 "blocks_n": block_decompose(info.n_pad) if info.block_diagonal else [info.n_pad]}
            if layer.glq_is_trellis:
                d["inv2"] = float(shard["inv_resid_scale2"].item()) if info.n_stages == 2 else 0.0
            else:
                d["inv"] = [float(shard[k].item()) if k in shard else 0.0 for k in _E8_SCALES]
            meta.append(d)
        layer.glq_meta = meta
        # the quantizer draws every layer's signs from the same seed, so the parts of a merged layer usually share SV
        # (then one input transform serves them all); checked here, once, because the comparison synchronises
        layer.glq_shared_sv = all(bufs["SV"].get_shard(i).shape == bufs["SV"].get_shard(0).shape and
                                  bool(torch.equal(bufs["SV"].get_shard(i), bufs["SV"].get_shard(0))) for i in range(1, len(meta)))
        if not layer.glq_is_trellis:
            layer.glq_cb = self.codebook.to(device=device, dtype=torch.float16)
            layer.glq_cb2 = (self.codebook2 if self.codebook2 is not None else self.codebook).to(device=device, dtype=torch.float16)
        layer.glq_reduce = (self.comm if (self.comm is not None and self.comm.world > 1 and layer.glq_row_parallel
                                          and getattr(layer, "glq_tp_sharded", False)) else None)
        layer.glq_ready = True
        x = torch.zeros(1, layer.glq_in_features, dtype=layer.glq_params_dtype, device=device)
        if layer.glq_reduce is None:          # a warm-up through a communicator would need every rank at this point
            self.apply(layer, x)
            torch.cuda.synchronize(device)

    # ---- apply ----------------------------------------------------------------------------------------------
    def apply(self, layer, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not getattr(layer, "glq_ready", False):
            raise RuntimeError("glq_b200: process_weights_after_loading has not run for this layer")
        shape = x.shape
        x2d = x.reshape(-1, layer.glq_in_features)
        bufs, meta = layer.glq_buffers, layer.glq_meta
        g = lambda name, i: bufs[name].get_shard(i)
        if layer.glq_is_trellis:
            if layer.glq_is_fused and layer.glq_shared_sv:
                # shards that share one input transform: one plan (one launch up to 8 tokens) for all of them
                y = ops.fused_linear_trellis_3inst_shards(
                    x2d, g("SV", 0), [(g("SU", i), g("trellis_packed", i), g("trellis_packed2", i) if m["n_stages"] == 2 else None,
                                       m["wscale"], m["inv2"], m["m"]) for i, m in enumerate(meta)])
            else:
                outs = []
                for i, m in enumerate(meta):
                    bn, bm = torch.tensor(m["blocks_n"]), torch.tensor(m["blocks_m"])
                    if m["n_stages"] == 2:
                        outs.append(ops.fused_linear_trellis_3inst_rvq2(
                            x2d, g("SV", i), g("SU", i), g("trellis_packed", i), g("trellis_packed2", i), bn, bm, None, None,
                            m["wscale"], m["inv2"], m["n_pad"], m["m"], m["n_pad"], m["m_pad"]))
                    else:
                        outs.append(ops.fused_linear_trellis_3inst(
                            x2d, g("SV", i), g("SU", i), g("trellis_packed", i), bn, bm, None, None, m["wscale"],
                            m["n_pad"], m["m"], m["n_pad"], m["m_pad"], reduce_over=layer.glq_reduce))
                y = outs[0] if len(outs) == 1 else torch.cat(outs, dim=-1)
        else:
            outs = []
            dev = x.device
            empty_i = torch.empty(0, dtype=torch.int16, device=dev)
            empty_h = torch.empty(0, dtype=torch.float16, device=dev)
            for i, m in enumerate(meta):
                ns, inv = m["n_stages"], m["inv"]
                tail = (g("Qidxs2", i) if ns >= 2 else empty_i, layer.glq_cb2 if ns >= 2 else empty_h, inv[0] if ns >= 2 else 0.0,
                        g("Qidxs3", i) if ns >= 3 else empty_i, layer.glq_cb if ns >= 3 else empty_h, inv[1] if ns >= 3 else 0.0,
                        g("Qidxs4", i) if ns >= 4 else empty_i, layer.glq_cb if ns >= 4 else empty_h, inv[2] if ns >= 4 else 0.0)
                if m["block_diagonal"]:
                    yi = ops.fused_linear_block_diag(x2d, g("SV", i), g("SU", i), g("Qidxs", i), layer.glq_cb, m["wscale"],
                                                     layer.glq_in_features, m["m"], m["n_pad"], m["m_pad"],
                                                     torch.tensor(m["blocks_n"]), torch.tensor(m["blocks_m"]), None, None, *tail)
                else:
                    yi = ops.fused_linear(x2d, g("SV", i), g("SU", i), g("Qidxs", i), layer.glq_cb, m["wscale"],
                                          layer.glq_in_features, m["m"], m["n_pad"], m["m_pad"],
                                          m["n_pad"].bit_length() - 1, m["m_pad"].bit_length() - 1, *tail)
                if layer.glq_reduce is not None:
                    yi32 = yi.float().contiguous()
                    if yi32.numel() <= layer.glq_reduce.max_floats:
                        layer.glq_reduce.all_reduce_(yi32)
                    else:
                        import torch.distributed as dist
                        dist.all_reduce(yi32)
                    yi = yi32.to(yi.dtype)
                outs.append(yi)
            y = outs[0] if len(outs) == 1 else torch.cat(outs, dim=-1)
        if bias is not None:
            y = y + bias.to(y.dtype)
        return y.reshape(*shape[:-1], y.shape[-1])
