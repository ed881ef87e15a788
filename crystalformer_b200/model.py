"""Model shell with the reference's interface and state_dict keys (models/latticeformer.py:32-302):
98-dim one-hot species -> Linear embedding -> encoder -> (optional projection) -> per-crystal pooling -> MLP head.
Only what the benchmark configurations use is implemented: ``pooling`` in {"avr", "max"}, ``pre_pooling_op`` in
{"no", "relu", "w+relu"}, ``norm_type`` in {"no", "id", "ln"}; the reference's single-process multi-GPU split is
replaced by one process per GPU (``crystalformer_b200.sharding``)."""
from __future__ import annotations

import copy
import ctypes
import types
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import _lib
from .cuda_funcs import IrregularMeanCUDA
from .encoder import BatchGeometry, CrystalformerEncoderCUDA, pack_dense_weight
from .params import DEFAULT_MODEL_PARAMS, LatticeformerParams


def default_params(**overrides) -> types.SimpleNamespace:
    """Attribute bag carrying the keys of the reference's params/latticeformer/default.json."""
    p = copy.deepcopy(DEFAULT_MODEL_PARAMS)
    p.update(overrides)
    return types.SimpleNamespace(**p)


def avr_pool(x, batch, sizes):
    """Deterministic per-crystal mean (models/pooling.py:19-25 with the CUDA branch)."""
    return IrregularMeanCUDA.apply(x, batch, sizes)


def max_pool(x, batch, sizes):
    """Per-crystal maximum (models/pooling.py:14-17), without the host loop."""
    B = sizes.shape[0]
    out = torch.full((B, x.shape[1]), float("-inf"), dtype=x.dtype, device=x.device)
    return out.scatter_reduce(0, batch[:, None].expand_as(x), x, reduce="amax", include_self=True)


class Latticeformer(nn.Module):
    def __init__(self, params):
        super().__init__()
        embedding_dim = copy.deepcopy(params.embedding_dim)
        self.params = params
        num_layers = getattr(params, "num_layers", 4)
        model_dim = getattr(params, "model_dim", 128)
        ff_dim = getattr(params, "ff_dim", 512)
        t_fixup_init = getattr(params, "t_fixup_init", True)
        self.pooling = getattr(params, "pooling", "max")
        pre_pooling_op = getattr(params, "pre_pooling_op", "w+bn+relu")
        dropout = getattr(params, "dropout", 0.1)
        head_num = getattr(params, "head_num", 8)
        v_dim = getattr(params, "v_dim", 0)
        k_dim = getattr(params, "k_dim", 0)
        norm_type = getattr(params, "norm_type", "bn")
        t_activation = getattr(params, "t_activation", "relu")
        if getattr(params, "use_cgcnn_feat", False) or getattr(params, "scale_grad", 0.0) > 0:
            raise NotImplementedError("use_cgcnn_feat / scale_grad are not supported")

        lattice_params = LatticeformerParams()
        lattice_params.parseFromArgs(params)

        self.ATOM_FEAT_DIM = 98
        self.input_embeddings = nn.Linear(self.ATOM_FEAT_DIM, model_dim, bias=False)
        emb_scale = model_dim ** (-0.5)
        if t_fixup_init:
            emb_scale *= (9 * num_layers) ** (-1 / 4)
        nn.init.normal_(self.input_embeddings.weight, mean=0, std=emb_scale)

        self.encoder = CrystalformerEncoderCUDA(
            model_dim, head_num, activation=t_activation, num_encoder_layers=num_layers, dim_feedforward=ff_dim,
            dropout=dropout, t_fixup_init=t_fixup_init, no_layer_norm=t_fixup_init, lattice_params=lattice_params,
            k_dim=k_dim, v_dim=v_dim)

        if norm_type == "ln":
            norm = nn.LayerNorm
        elif norm_type in ("id", "no"):
            norm = nn.Identity
        else:
            raise NotImplementedError(f"norm_type: {norm_type}")

        dim_pooled = model_dim
        self.proj_before_pooling = lambda x: x
        if pre_pooling_op == "w+relu":
            dim_pooled = embedding_dim.pop(0)
            self.proj_before_pooling = nn.Sequential(nn.Linear(model_dim, dim_pooled), nn.ReLU(True))
        elif pre_pooling_op == "relu":
            self.proj_before_pooling = nn.ReLU(True)
        elif pre_pooling_op != "no":
            raise NotImplementedError(f"pre_pooling_op: {pre_pooling_op}")

        if self.pooling == "max":
            self.pooling_layer = max_pool
        elif self.pooling == "avr":
            self.pooling_layer = avr_pool
        else:
            raise NotImplementedError(f"pooling: {self.pooling}")

        final_dim = 1 if isinstance(params.targets, str) else len(params.targets)
        in_dim = [dim_pooled] + embedding_dim[:-1]
        layers = []
        for di, do in zip(in_dim, embedding_dim):
            layers += [nn.Linear(di, do), norm(do), nn.ReLU(True)]
        layers.append(nn.Linear(embedding_dim[-1], final_dim))
        self.mlp = nn.Sequential(*layers)

    # ---------------------------------------------------------------------------------------------------------------
    # Inference fast path: embedding, geometry, encoder, pooling and head in one call into the library
    # (cf_model_forward); taken in eval mode without autograd when the configuration is the one it implements.
    # ---------------------------------------------------------------------------------------------------------------
    def _native_ok(self) -> bool:
        if not getattr(self, "native", True) or self.pooling != "avr" or isinstance(self.proj_before_pooling, nn.Module):
            return False
        m = self.mlp
        if not (len(m) == 4 and isinstance(m[0], nn.Linear) and isinstance(m[1], nn.Identity)
                and isinstance(m[2], nn.ReLU) and isinstance(m[3], nn.Linear) and m[0].in_features == 128
                and m[0].out_features <= 1024 and m[0].bias is not None and m[3].bias is not None):
            return False
        return self.input_embeddings.out_features == 128 and self.encoder.native and self.encoder._native_ok()

    def _embedding_packed(self, device) -> Optional[torch.Tensor]:
        """The embedding weight, input columns zero-padded to 128, in the fragment order of the fused dense kernel
        (which then computes the embedding inside the encoder's first launch); None when that kernel is not in use.
        Rebuilt only when the weight changed."""
        W = self.input_embeddings.weight
        if not self.encoder.dense_fused or W.shape[1] > 128:
            return None
        key = (device, W._version, W.data_ptr())
        cache = getattr(self, "_embed_cache", None)
        if cache is None or cache[0] != key:
            padded = torch.zeros((128, 128), dtype=torch.float32, device=device)
            padded[:, :W.shape[1]] = W.detach().float()
            self._embed_cache = cache = (key, pack_dense_weight(padded))
        return cache[1]

    def native_plan(self, device) -> dict:
        """Everything of a native forward that does not depend on the batch: packed encoder weights, the head's weights
        as contiguous float32 tensors, the packed embedding and the scalar arguments of cf_model_forward.  Building it
        checks every parameter's version; a caller that runs many batches through unchanged weights (the serving
        pipeline) builds it once and hands it to ``_forward_native``."""
        enc = self.encoder
        P = enc.lattice_params
        f32 = lambda t: t.detach().float().contiguous()
        w = enc._packed_weights(device)
        plan = dict(w=w, emb=f32(self.input_embeddings.weight), w1=f32(self.mlp[0].weight), b1=f32(self.mlp[0].bias),
                    w2=f32(self.mlp[3].weight), b2=f32(self.mlp[3].bias), emb_packed=self._embedding_packed(device))
        dist_max = P.value_pe_dist_max
        if dist_max < 0:
            sr = P.scale_real[0] if isinstance(P.scale_real, (list, tuple)) else P.scale_real
            dist_max = -dist_max * sr
        plan["hidden"], plan["targets"] = plan["w1"].shape[0], plan["w2"].shape[0]
        if plan["emb_packed"] is not None:  # the description of the model for cf_serve_submit
            plan["desc"] = _lib.ModelDesc(
                feature_dim=plan["emb"].shape[1], W_embed=plan["emb"].data_ptr(), W_embed_packed=plan["emb_packed"].data_ptr(),
                num_layers=len(enc.layers), lattice_range=int(P.lattice_range),
                minimum_range=int(P.lattice_range) if P.minimum_range else 0, dense_tile_rows=0,
                weights=ctypes.cast(w["ptrs"], ctypes.c_void_p), scalars=ctypes.cast(w["scalars"], ctypes.c_void_p),
                K=int(P.value_pe_dist_real), ff_dim=w["ff"], wscale=float(P.value_pe_width_scale), cutoff_radius=enc._cutoff(),
                W1=plan["w1"].data_ptr(), b1=plan["b1"].data_ptr(), hidden=plan["hidden"], W2=plan["w2"].data_ptr(),
                b2=plan["b2"].data_ptr(), targets=plan["targets"], order_reach=float(dist_max) + 1.0)
        plan["tail"] = (len(enc.layers), w["ptrs"], w["scalars"], int(P.value_pe_dist_real), w["ff"],
                        float(P.value_pe_width_scale), enc._cutoff(), int(P.lattice_range),
                        int(P.lattice_range) if P.minimum_range else 0, plan["w1"].data_ptr(), plan["b1"].data_ptr(),
                        plan["hidden"], plan["w2"].data_ptr(), plan["b2"].data_ptr(), plan["targets"], float(dist_max) + 1.0)
        return plan

    WORKSPACE_RING = 4  # forwards whose preparation may be in flight at a time (see _forward_native, inputs_ready)

    def _ring_workspace(self, dev, nbytes: int):
        """Next workspace of a small ring of persistent buffers, with the event that marks the end of its previous use:
        a forward whose preparation starts early (``inputs_ready``) runs beside the forwards before it, so it cannot
        share their scratch memory."""
        ring = getattr(self, "_ws_ring", None)
        if ring is None or ring["dev"] != dev:
            ring = self._ws_ring = dict(dev=dev, slots=[None] * self.WORKSPACE_RING, next=0)
        at = ring["next"] % self.WORKSPACE_RING
        ring["next"] += 1
        slot = ring["slots"][at]
        if slot is None or slot[0].numel() < nbytes:
            slot = ring["slots"][at] = [torch.empty(nbytes, dtype=torch.uint8, device=dev), torch.cuda.Event(), False]
        return slot

    def _forward_native(self, data, counts: Tuple[int, int, int], gather=None, plan: Optional[dict] = None,
                        inputs_ready: Optional[torch.cuda.Event] = None) -> torch.Tensor:
        dev = data.pos.device
        if plan is None:
            plan = self.native_plan(dev)
        n_atoms, n_edges, max_atoms = (int(v) for v in counts)
        f32 = lambda t: t if (t.dtype == torch.float32 and t.is_contiguous()) else t.detach().float().contiguous()
        feats, pos, trans = f32(data.x), f32(data.pos), f32(data.trans_vec)
        sizes = data.sizes
        if sizes.device != dev or sizes.dtype != torch.int64 or not sizes.is_contiguous():
            sizes = sizes.to(device=dev, dtype=torch.int64).contiguous()
        B = sizes.shape[0]
        lib = _lib.load()
        ff = plan["w"]["ff"]
        nbytes = int(lib.cf_model_workspace_bytes(n_atoms, B, n_edges, ff))
        emb_packed = plan["emb_packed"]
        slot = None
        if inputs_ready is not None and emb_packed is not None:
            slot = self._ring_workspace(dev, nbytes)
            work = slot[0]
        else:
            work = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        y = torch.empty((B, plan["targets"]), dtype=torch.float32, device=dev)
        desc = None if gather is None else gather.next_descriptor()
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev)
            if slot is not None and slot[2]:
                stream.wait_event(slot[1])  # (a no-op in effect unless the workspace was last used on another stream)
            _lib.call("cf_model_forward", ctypes.c_void_p(torch.cuda.current_blas_handle()),
                      feats.data_ptr(), feats.shape[1], pos.data_ptr(), trans.data_ptr(), sizes.data_ptr(), n_atoms, B,
                      n_edges, max_atoms, plan["emb"].data_ptr(), None if emb_packed is None else emb_packed.data_ptr(),
                      *plan["tail"], work.data_ptr(), y.data_ptr(), self.encoder._attention_events(),
                      None if desc is None else ctypes.byref(desc),
                      None if slot is None else ctypes.c_void_p(inputs_ready.cuda_event),
                      None if (slot is None or not slot[2]) else ctypes.c_void_p(slot[1].cuda_event), stream.cuda_stream)
            if slot is not None:
                slot[1].record(stream)  # the next forward that takes this workspace waits for this one
                slot[2] = True
        return y if gather is None else gather.collect()

    def forward(self, data, geometry: Optional[BatchGeometry] = None, counts: Optional[Tuple[int, int, int]] = None,
                gather=None, inputs_ready: Optional[torch.cuda.Event] = None):
        """``data`` carries x (N,98), pos (N,3), batch (N), trans_vec (B,3,3), sizes (B) like the reference's PyG batch.
        ``counts`` = (atoms, edges = sum n^2, largest crystal), when the caller knows them on the host, saves the
        device->host read of ``sizes``.  ``gather`` (a ``sharding.PeerGather``, inference only): the outputs of every
        rank's crystals are returned, in the order of the unsharded batch.  ``inputs_ready`` (inference through the
        one-call path only): a CUDA event after which the tensors of ``data`` are valid.  The batch preparation, which
        depends on the inputs alone, is then not ordered behind the work already queued on the current stream and
        overlaps the previous batch's forward; the tensors must stay unchanged until this forward has run."""
        if geometry is None and not self.training and not torch.is_grad_enabled() and data.pos.is_cuda \
                and self._native_ok():
            if counts is None:
                host = data.sizes.tolist()  # the one device->host read per batch (the reference does the same)
                counts = (sum(host), sum(n * n for n in host), max(host) if host else 1)
            return self._forward_native(data, counts, gather, inputs_ready=inputs_ready)
        x = self.input_embeddings(data.x)
        if geometry is None:
            geometry = BatchGeometry(data.pos, data.trans_vec, data.sizes, *(counts if counts is not None else ()))
        g = geometry
        x = self.encoder(x, data.pos, g.batch, data.trans_vec, g.sizes, geometry=g)
        x = self.proj_before_pooling(x)
        x = self.pooling_layer(x, g.batch, g.sizes)
        y = self.mlp(x)
        if gather is not None:
            gather.store(y)
            return gather.collect()
        return y
