"""Model-level harness: the reference's AutoFocusFormer, unmodified, calling this package's operators.

The CLUSTEN operators are called from three lines of models/aff_transformer.py of
apple/ml-autofocusformer (:120 QK, :154 AV, :361 WF).  This module imports that file as it
is (sourceless bytecode that oracle/build_ref.py compiles from the checkout into
oracle/_ref/aff_model/; nothing of the model is re-implemented here) and supplies the three
things the file needs that are not in this environment:

  * `timm.models.layers.DropPath` / `trunc_normal_` (models/aff_transformer.py:9): written
    here from their documented behaviour -- DropPath is the identity in eval mode and, in
    training, zeroes whole samples with probability p and rescales the rest by 1 / (1 - p);
    trunc_normal_ is torch.nn.init.trunc_normal_.
  * `knn_keops` (models/point_utils.py:27-58; pykeops is not installed): the k nearest
    database points of every query by exact Euclidean distance, ascending: on the GPU the
    library's clusten_knn2d kernel, on the CPU torch.cdist + topk.  Tie-breaking of the
    original is not pinned by any reference test.
  * the `clusten` package: this repository's operators ("b200"), the PyTorch gather
    formulation of the reference's kernel tests ("formula", the parity checker), or the
    reference's own wrappers on its own CUDA kernels ("reference", the speed bar).

The same stand-ins serve every implementation, so a comparison between two of them is a
comparison of the operators on identical neighbourhood tables.

Configurations (BASELINE configs 3 and 4):
  tiny224  embed 64/128/256/512, depths 2/2/6/2, heads 2/4/8/16, mlp_ratio 3 (configs/aff_tiny.yaml:7-8),
           cluster 8, nbhd 48/48/48/49, ds_rate 1/4, 224 x 224 input, 1000 classes
  base384  embed 128/256/512/1024, depths 3/4/18/2, heads 4/8/16/32, mlp_ratio 3, layer_scale 1e-5
           (configs/aff_base_22kto1k_384.yaml:6-12), cluster 8, nbhd 48/48/48/49, ds_rate 1/5, 384 x 384
"""
import importlib
import importlib.machinery
import importlib.util
import math
import os
import sys
import types

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_REF = os.path.join(_ROOT, "oracle", "_ref")
MODEL_DIR = os.path.join(_REF, "aff_model")
REF_CLUSTEN_DIR = os.path.join(_REF, "ref_clusten")

CONFIGS = {
    "tiny224": dict(embed_dim=[64, 128, 256, 512], depths=[2, 2, 6, 2], num_heads=[2, 4, 8, 16], mlp_ratio=3.,
                    cluster_size=8, nbhd_size=[48, 48, 48, 49], ds_rate=0.25, layer_scale=0.0, img_size=224,
                    num_classes=1000, drop_path_rate=0.0),
    "base384": dict(embed_dim=[128, 256, 512, 1024], depths=[3, 4, 18, 2], num_heads=[4, 8, 16, 32], mlp_ratio=3.,
                    cluster_size=8, nbhd_size=[48, 48, 48, 49], ds_rate=0.2, layer_scale=1e-5, img_size=384,
                    num_classes=1000, drop_path_rate=0.0),
}


def available():
    """Is the reference's model bytecode there (oracle/build_ref.py has run)?"""
    return os.path.exists(os.path.join(MODEL_DIR, "models", "aff_transformer.bytecode"))


def _load_bytecode(name, path):
    """Import the sourceless module stored at `path` (.pyc format) as `name`."""
    loader = importlib.machinery.SourcelessFileLoader(name, path)
    spec = importlib.util.spec_from_loader(name, loader, origin=path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    try:
        loader.exec_module(mod)
    except BaseException:
        sys.modules.pop(name, None)
        raise
    return mod


# ----------------------------------------------------------------------------- stand-ins
class DropPath(torch.nn.Module):
    """Stochastic depth per sample: identity in eval mode or with p = 0."""

    def __init__(self, drop_prob=0.0):
        super().__init__()
        self.drop_prob = float(drop_prob)

    def forward(self, x):
        if self.drop_prob == 0.0 or not self.training:
            return x
        keep = 1.0 - self.drop_prob
        mask = x.new_empty((x.shape[0],) + (1,) * (x.dim() - 1)).bernoulli_(keep)
        return x * mask / keep


def _install_timm_standin():
    if "timm.models.layers" in sys.modules:
        return
    try:
        importlib.import_module("timm.models.layers")
        return
    except ImportError:
        pass
    timm = types.ModuleType("timm")
    models = types.ModuleType("timm.models")
    layers = types.ModuleType("timm.models.layers")
    layers.DropPath = DropPath
    layers.trunc_normal_ = torch.nn.init.trunc_normal_
    timm.models, models.layers = models, layers
    sys.modules.update({"timm": timm, "timm.models": models, "timm.models.layers": layers})


def knn(query, database, k, return_dist=False, chunk_elems=1 << 28):
    """Interface of knn_keops (models/point_utils.py:27-58): query [b, n_, d], database [b, n, d]
    -> indices [b, n_, k] of the k nearest database points by ascending distance (and the distances).
    Exact fp32 distances (no matrix-multiply shortcut); batches are processed in chunks so that the
    [chunk, n_, n] distance matrix stays below chunk_elems elements."""
    with torch.no_grad():
        q = query.detach().float()
        d = database.detach().float()
        if q.is_cuda and q.shape[2] == 2 and k <= 8 and k <= d.shape[1] and q.shape[0] <= 65535:
            # on the GPU the search is the library's kernel (clusten_knn2d): same definition, ties towards the
            # lower index
            from clusten import ops
            return ops.knn2d(q.contiguous(), d.contiguous(), k, return_dist)
        b, nq, _ = q.shape
        n = d.shape[1]
        step = max(1, min(b, chunk_elems // max(1, nq * n)))
        idxs, dists = [], []
        for s in range(0, b, step):
            dist = torch.cdist(q[s:s + step], d[s:s + step], compute_mode="donot_use_mm_for_euclid_dist")
            nn_dist, nn_idx = dist.topk(k, dim=2, largest=False, sorted=True)
            idxs.append(nn_idx)
            dists.append(nn_dist)
        nn_idx = torch.cat(idxs, 0)
        if return_dist:
            return nn_idx, torch.cat(dists, 0)
        return nn_idx


# ----------------------------------------------------------------------------- clusten implementations
class _FormulaFunction:
    """`.apply(a, b, nbhd_idx)` on the PyTorch gather formulation (oracle/formula.py), with the
    operators' dtype rule: the second tensor is converted to the first one's dtype."""

    def __init__(self, fn, chunk):
        self.fn, self.chunk = fn, chunk

    def apply(self, a, b, nbhd_idx):
        b = b.to(a.dtype)
        step = self.chunk
        if step is None or step >= a.shape[0]:
            return self.fn(a, b, nbhd_idx)
        return torch.cat([self.fn(a[s:s + step], b[s:s + step], nbhd_idx[s:s + step])
                          for s in range(0, a.shape[0], step)], 0)


def _implementation(name, formula_chunk=8):
    """-> (CLUSTENQKFunction, CLUSTENAVFunction, CLUSTENWFFunction) of the named implementation."""
    if name == "b200":
        import clusten
        return clusten.CLUSTENQKFunction, clusten.CLUSTENAVFunction, clusten.CLUSTENWFFunction
    if name == "formula":
        if _ROOT not in sys.path:
            sys.path.insert(0, _ROOT)
        from oracle import formula
        return (_FormulaFunction(formula.qk, formula_chunk), _FormulaFunction(formula.av, formula_chunk),
                _FormulaFunction(formula.wf, formula_chunk))
    if name == "reference":
        # the reference's clusten/clusten.py (bytecode) on its own extension modules in oracle/_ref/
        if _REF not in sys.path:
            sys.path.insert(0, _REF)
        mod = sys.modules.get("reference_clusten_wrappers") or _load_bytecode(
            "reference_clusten_wrappers", os.path.join(REF_CLUSTEN_DIR, "clusten", "clusten.bytecode"))
        return mod.CLUSTENQKFunction, mod.CLUSTENAVFunction, mod.CLUSTENWFFunction
    raise ValueError(name)


def reference_kernels_available():
    if not os.path.exists(os.path.join(REF_CLUSTEN_DIR, "clusten", "clusten.bytecode")):
        return False
    try:
        _implementation("reference")
        return True
    except Exception:
        return False


_aff = None


def model_module():
    """The reference's models.aff_transformer, imported once with the stand-ins in place."""
    global _aff
    if _aff is None:
        if not available():
            raise RuntimeError("the reference model's bytecode is missing: run oracle/build_ref.py where the "
                               "checkout of apple/ml-autofocusformer is present")
        _install_timm_standin()
        import clusten  # noqa: F401  this package's operators: what `from clusten import ...` in the model resolves to
        # a package `models` holding exactly the two modules of the measured path
        pkg_dir = os.path.join(MODEL_DIR, "models")
        pkg = types.ModuleType("models")
        pkg.__path__ = [pkg_dir]
        sys.modules["models"] = pkg
        point_utils = _load_bytecode("models.point_utils", os.path.join(pkg_dir, "point_utils.bytecode"))
        point_utils.knn_keops = knn
        pkg.point_utils = point_utils
        _aff = _load_bytecode("models.aff_transformer", os.path.join(pkg_dir, "aff_transformer.bytecode"))
        _aff.knn_keops = knn
        pkg.aff_transformer = _aff
    return _aff


def use_implementation(name, **kw):
    """Make the model's three call sites use the named `clusten` implementation."""
    aff = model_module()
    aff.CLUSTENQKFunction, aff.CLUSTENAVFunction, aff.CLUSTENWFFunction = _implementation(name, **kw)
    return aff


_original_attention_forward = None


def _fused_cluster_attention_forward(self, feat, member_idx, cluster_mask, pe_idx, global_attn):
    """ClusterAttention.forward (models/aff_transformer.py:85-160 of the reference) with the local-attention
    chain -- QK :120, position embedding :129-134, mask :136-137, blank token :140-141, softmax :142, AV :154,
    blank value :147,155 -- done by one call of the library's fused kernel.  Same parameters, same Linear
    layers before and after; global attention (the last stage at 224 x 224) keeps the original code."""
    if global_attn:
        return _original_attention_forward(self, feat, member_idx, cluster_mask, pe_idx, global_attn)
    from clusten import ops
    aff = model_module()
    b, n, c = feat.shape
    h = self.num_heads
    c_ = c // h
    q = self.q(feat) * self.scale                                   # b x n x c
    kv = self.kv(feat)                                              # b x n x 2c
    q = q.reshape(b, n, h, -1).permute(0, 2, 1, 3)                  # b x h x n x c_ (view)
    kv = kv.view(b, n, h, 2, c_).permute(3, 0, 2, 1, 4)             # 2 x b x h x n x c_ (views)
    if not aff.pre_table.is_cuda:
        aff.pre_table = aff.pre_table.to(pe_idx.device)
    pe_table = self.pos_embed(aff.pre_table).to(q.dtype)            # table rows x h
    out = ops.local_attention_forward(
        q, kv[0], kv[1], member_idx.contiguous(), pe_table=pe_table.contiguous(), pe_idx=pe_idx.contiguous(),
        mask=None if cluster_mask is None else cluster_mask.contiguous(),
        blank_k=self.blank_k.reshape(h, c_).to(q.dtype).contiguous(),
        blank_v=self.blank_v.reshape(h, c_).to(q.dtype).contiguous())
    out = out.permute(0, 2, 1, 3).reshape(b, n, c)
    return self.proj_drop(self.proj(out))


def use_fused_attention(on=True):
    """Opt-in: route ClusterAttention through the fused local-attention kernel (inference only).  This replaces
    one method of the reference's model, so figures taken with it are reported beside, never instead of, the
    figures of the unmodified model."""
    global _original_attention_forward
    aff = model_module()
    if _original_attention_forward is None:
        _original_attention_forward = aff.ClusterAttention.forward
    aff.ClusterAttention.forward = _fused_cluster_attention_forward if on else _original_attention_forward


_original_layer_forward = None


def _fused_basic_layer_forward(self, pos, feat, h, w, on_grid, stride):
    """BasicLayer.forward (models/aff_transformer.py:428-505 of the reference) with the stage's neighbourhood
    tables -- members of the nearest clusters :479, their mask :481-482, offsets and position-table rows
    :483-487 -- built by one call of the library instead of three gathers and the arithmetic between them.
    Clustering, the nearest-cluster search, the blocks and the merge are the reference's; stages with global
    attention or one-token clusters keep the original code."""
    b, n, d = pos.shape
    cs = self.cluster_size
    k = int(math.ceil(n / float(cs)))
    if self.nbhd_size >= n or k == n or d != 2 or pos.dtype != torch.float32:
        return _original_layer_forward(self, pos, feat, h, w, on_grid, stride)
    from clusten import ops
    aff = model_module()
    c = feat.shape[2]
    nnc = min(int(round(self.nbhd_size / float(cs))), k)
    self.nbhd_size = cs * nnc
    if on_grid:
        # the first feature map is the same grid for every image: clustered once, kept on the layer
        if self.cluster_mean_pos is None:
            (self.pos, self.cluster_mean_pos, self.member_idx, self.cluster_mask,
             self.reorder) = aff.space_filling_cluster(pos, cs, h, w, no_reorder=False)
        pos, means, members, reorder = self.pos[:b], self.cluster_mean_pos[:b], self.member_idx[:b], self.reorder[:b]
        cmask = None if self.cluster_mask is None else self.cluster_mask[:b]
    else:
        pos, means, members, cmask, reorder = aff.space_filling_cluster(pos, cs, h, w, no_reorder=False)
    feat = feat.gather(1, reorder.reshape(b, n, 1).expand(-1, -1, c))     # the tokens of a cluster side by side
    nearest = aff.knn_keops(pos, means, nnc)
    member_idx, cluster_mask, pe_idx = ops.nbhd_build(
        pos.contiguous(), members.contiguous(), None if cmask is None else cmask.contiguous(), nearest.contiguous(),
        aff.rel_pos_width, aff.table_width)
    for blk in self.blocks:
        feat = blk(feat=feat, member_idx=member_idx, cluster_mask=cluster_mask, pe_idx=pe_idx, global_attn=False)
    if self.downsample is not None:
        learned_prob = self.prob_net(feat).sigmoid()
        reserve_num = math.ceil(h / (stride * 2)) * math.ceil(w / (stride * 2))
        pos, feat = self.downsample(pos=pos, feat=feat, member_idx=member_idx, cluster_mask=cluster_mask,
                                    learned_prob=learned_prob, stride=stride, pe_idx=pe_idx, reserve_num=reserve_num)
    return pos, feat


def use_fused_neighbourhood(on=True):
    """Opt-in: build every stage's neighbourhood tables with clusten_nbhd_build.  Like use_fused_attention this
    replaces one method of the reference's model; its figures are reported beside the unmodified model's."""
    global _original_layer_forward
    aff = model_module()
    if _original_layer_forward is None:
        _original_layer_forward = aff.BasicLayer.forward
    aff.BasicLayer.forward = _fused_basic_layer_forward if on else _original_layer_forward


_original_merging_forward = None


def _fused_cluster_merging_forward(self, pos, feat, member_idx, cluster_mask, learned_prob, stride, pe_idx,
                                   reserve_num):
    """ClusterMerging.forward (models/aff_transformer.py:276-365 of the reference) with the merge weights --
    table rows by pe_idx :347-350, importance scores of the neighbours :340, mask and products :352-358 --
    formed by one call of the library.  Choosing the merge centres (:294-331) and everything after CLUSTENWF
    are the reference's computation, restated."""
    from clusten import ops
    aff = model_module()
    b, n, c = feat.shape
    d = pos.shape[2]
    keep = int(n * self.ds_rate)
    # ---- merge centres: tokens on the (adaptive) coarse lattice first, then by importance score
    if stride == 2:
        on_lattice = ((pos % stride).sum(-1) == 0).float()
    else:
        _, spacing = aff.knn_keops(pos, pos, 2, return_dist=True)
        spacing = 2 ** (spacing[:, :, 1].log2().ceil() + 1)
        on_lattice = ((pos.long() % spacing.unsqueeze(2).long()).sum(-1) == 0).float()
    score = on_lattice
    if learned_prob is not None:
        score = score + learned_prob.detach().view(b, n) * self.alpha
    if self.reserve_on:
        reserved = ((pos % (stride * 2)).sum(-1) == 0).float()
        score = score + reserved * (-100)
        picked = score.topk(keep - reserve_num, dim=1, sorted=False)[1]
        centres = torch.cat([picked, reserved.nonzero(as_tuple=True)[1].reshape(b, reserve_num)], dim=-1)
    else:
        centres = score.topk(keep, dim=1, sorted=False)[1]
    if centres.shape[1] != keep:
        raise RuntimeError("the number of merge centres differs from the number of tokens to keep")
    # ---- the centres' rows of the stage's tables
    row = centres.unsqueeze(2)
    m = member_idx.shape[-1]
    pos = pos.gather(1, row.expand(-1, -1, d))
    member_idx = member_idx.gather(1, row.expand(-1, -1, m))
    pe_idx = pe_idx.gather(1, row.expand(-1, -1, m))
    if cluster_mask is not None:
        cluster_mask = cluster_mask.gather(1, row.expand(-1, -1, m))
    # ---- merge weights, merge, projection
    if not aff.pre_table.is_cuda:
        aff.pre_table = aff.pre_table.to(pe_idx.device)
    weights = ops.merge_weights(self.weight_net(aff.pre_table), pe_idx, learned_prob, member_idx, cluster_mask)
    feat = aff.CLUSTENWFFunction.apply(weights, feat, member_idx).reshape(b, keep, -1)
    return pos, self.linear(self.norm(feat))


def use_fused_merging(on=True):
    """Opt-in: form ClusterMerging's weights with clusten_merge_weights (one method of the reference's model
    replaced; figures reported beside the unmodified model's)."""
    global _original_merging_forward
    aff = model_module()
    if _original_merging_forward is None:
        _original_merging_forward = aff.ClusterMerging.forward
    aff.ClusterMerging.forward = _fused_cluster_merging_forward if on else _original_merging_forward


def use_fused(on=True):
    """All three opt-ins together: fused attention, neighbourhood tables and merge weights from the library."""
    use_fused_attention(on)
    use_fused_neighbourhood(on)
    use_fused_merging(on)


def build_model(config, device, seed=0, **overrides):
    """AutoFocusFormer(**CONFIGS[config]).eval() with seeded random weights on `device`; keyword arguments
    replace entries of the configuration (e.g. reserve_on=False)."""
    aff = model_module()
    torch.manual_seed(seed)
    model = aff.AutoFocusFormer(**dict(CONFIGS[config], **overrides))
    return model.to(device).eval()


def synthetic_images(config, batch, device, seed=1):
    """N(0,1) images of the configuration's ImageNet shape (the dataset itself is not available)."""
    size = CONFIGS[config]["img_size"]
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn(batch, 3, size, size, generator=g, device=device)


def forward(model, images, dtype=torch.float32):
    """One inference forward the way main.py:343-354 of the reference runs it: no_grad, with
    autocast when a 16-bit dtype is asked for."""
    with torch.no_grad():
        if dtype == torch.float32:
            return model(images)
        with torch.autocast(device_type=images.device.type, dtype=dtype):
            return model(images)
