"""Regenerates the golden fixtures in this directory from the reference itself.

Run where the reference checkout is importable (it is pure Python on these
paths, CPU only):

    python tests/golden/make_golden.py /path/to/ResKV

It imports the reference's own ``reskv`` package and records, for small seeded
inputs, the outputs of the functions that run without a GPU:

* ``reskv.compression._encode``      unstructured FP16 encoder (K and V flavour)
* ``reskv.reference.reconstruct``    decoder of every bit layout
* ``reskv.reference.reference_attention`` / ``rotate``
* ``reskv.compression.cluster``      K-path Lloyd iterations
* ``reskv.compression._incremental_cluster``
* ``reskv.config.ResKVKernelConfig.resolve`` for the whole settings grid

The packers that exist only as CUDA kernels in the reference cannot be run
here; for those the CPU restatement (``oracle.encode``) produces the packed
words and the *reference's decoder* turns them back into dense tensors, which
is what gets stored.

The fixtures are consumed by ``tests/test_oracle_golden.py`` (oracle vs
reference) and by the GPU parity tests (CUDA vs the same vectors).
"""

from __future__ import annotations

import itertools
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent


def mixture(rng, b, h, t, clusters=8, sigma=0.3, outliers=True):
    """Seeded cluster-mixture K/V stand-in: centres N(0,1), within-cluster
    sigma, log-normal per-channel scales."""
    centres = rng.standard_normal((b, h, clusters, 128)).astype(np.float32)
    which = rng.integers(0, clusters, (b, h, t))
    x = np.take_along_axis(centres, np.broadcast_to(which[..., None], (b, h, t, 128)), axis=2)
    x = x + sigma * rng.standard_normal((b, h, t, 128)).astype(np.float32)
    if outliers:
        x = x * np.exp(rng.standard_normal((b, h, 1, 128))).astype(np.float32)
    return x.astype(np.float16)


def main(ref_root: str):
    sys.path.insert(0, str(ROOT))   # the oracle package
    sys.path.insert(0, ref_root)    # first: `reskv` must be the reference, not this repository's alias package
    import reskv.compression as rc
    if Path(rc.__file__).resolve().is_relative_to(ROOT / "reskv"):
        sys.exit("`reskv` resolved to this repository's alias package; pass the path of the reference checkout")
    import reskv.reference as rr
    from reskv.config import KernelPlan, ResKVKernelConfig
    from reskv.tensors import CompressedKV, CompressedTensor

    from oracle import encode as oenc

    torch.set_num_threads(1)
    out = {}
    rng = np.random.default_rng(20240607)

    # ---- inputs shared by the encoder / decoder / attention cases ----------
    b, h, t, c = 1, 2, 96, 8
    x_k = mixture(rng, b, h, t)
    x_v = mixture(rng, b, h, t)
    cen_k = (rng.standard_normal((b, h, c, 128)) * 0.5).astype(np.float16)
    cen_v = (rng.standard_normal((b, h, c, 128)) * 0.5).astype(np.float16)
    ids_k = rng.integers(0, c, (b, h, t)).astype(np.int32)
    ids_v = rng.integers(0, c, (b, h, t)).astype(np.int32)
    # tie-free variant: residual magnitudes are a permutation of distinct values
    perm = np.argsort(rng.random((b, h, t, 128)), axis=-1)
    signs = rng.choice([-1.0, 1.0], (b, h, t, 128))
    x_distinct = ((perm + 1) * 0.125 * signs).astype(np.float16)
    zero_cen = np.zeros((b, h, 1, 128), np.float16)
    zero_ids = np.zeros((b, h, t), np.int32)
    out.update(x_k=x_k, x_v=x_v, cen_k=cen_k, cen_v=cen_v, ids_k=ids_k, ids_v=ids_v,
               x_distinct=x_distinct, zero_cen=zero_cen, zero_ids=zero_ids)

    T = torch.from_numpy

    def plan_for(layout, bits, nnz):
        fusion = {"unstructured": "deferred" if bits == 16 else "per_token", "tiled": "per_token",
                  "structured": "deferred"}[layout]
        return KernelPlan(layout, fusion, bits, nnz, 4, 0)

    # ---- 1. the reference's own unstructured FP16 encoder -------------------
    for nnz in (32, 64):
        plan = plan_for("unstructured", 16, nnz)
        for tag, x, cen, ids in (("k", x_k, cen_k, ids_k), ("v", x_v, cen_v, ids_v),
                                 ("d", x_distinct, zero_cen, zero_ids)):
            for value in (False, True):
                ct = rc._encode(T(x), T(cen), T(ids), plan, value=value)
                key = f"enc_u16_{tag}_{nnz}_{'v' if value else 'k'}"
                out[key + "_payload"] = ct.payload.numpy()
                out[key + "_meta"] = ct.metadata.numpy()

    # ---- 2. every layout through the reference's decoder --------------------
    layouts = [("unstructured", 16, 32), ("unstructured", 16, 64), ("tiled", 16, 64),
               ("structured", 16, 32), ("structured", 4, 32), ("unstructured", 4, 32),
               ("unstructured", 4, 64), ("unstructured", 2, 32), ("unstructured", 2, 64)]
    for layout, bits, nnz in layouts:
        plan = plan_for(layout, bits, nnz)
        p, m, s = oenc.encode(layout, bits, nnz, x_k, cen_k, ids_k)
        ct = CompressedTensor(T(cen_k), T(ids_k), T(p), T(m) if m is not None else None,
                              T(s) if s is not None else None, plan)
        key = f"dec_{layout}_{bits}_{nnz}"
        out[key + "_payload"] = p
        if m is not None:
            out[key + "_meta"] = m
        if s is not None:
            out[key + "_scale"] = s
        out[key + "_dense"] = rr.reconstruct(ct).numpy()

    # ---- 3. reference_attention ---------------------------------------------
    q = (rng.standard_normal((b, h * 4, 1, 128))).astype(np.float16)
    out["q"] = q
    freq_model = (500000.0 ** (-torch.arange(64).float() / 64) / torch.linspace(1, 8, 64)).numpy()
    out["freq_model"] = freq_model
    for nnz in (32, 64):
        plan = plan_for("unstructured", 16, nnz)
        k = rc._encode(T(x_k), T(cen_k), T(ids_k), plan)
        v = rc._encode(T(x_v), T(cen_v), T(ids_v), plan, value=True)
        cache = CompressedKV(k, v)
        out[f"att_{nnz}_theta"] = rr.reference_attention(T(q), cache, position=t + 40).numpy()
        out[f"att_{nnz}_freq_start"] = rr.reference_attention(
            T(q), cache, position=t + 40, start_position=7, inv_freq=T(freq_model), scaling=0.11).numpy()
        qr = rr.rotate(T(q), torch.tensor([t + 40]), T(freq_model)).half()
        kr = T((rng.standard_normal((b, h, 33, 128)) * 0.5).astype(np.float16))
        vr = T((rng.standard_normal((b, h, 33, 128)) * 0.5).astype(np.float16))
        out[f"att_{nnz}_qr"], out[f"att_{nnz}_kr"], out[f"att_{nnz}_vr"] = qr.numpy(), kr.numpy(), vr.numpy()
        out[f"att_{nnz}_recent"] = rr.reference_attention(
            T(q), cache, position=t + 40, inv_freq=T(freq_model), recent=(qr, kr, vr)).numpy()
    out["rotate_q"] = rr.rotate(T(q), torch.tensor([12345]), T(freq_model)).numpy()

    # ---- 4. Lloyd iterations, K path ----------------------------------------
    xk = mixture(rng, 1, 2, 512, clusters=6)
    out["km_x"] = xk
    for count, iters in ((8, 1), (8, 4), (32, 3)):
        cen, ids = rc.cluster(T(xk), count, iters)
        out[f"km_{count}_{iters}_centres"] = cen.numpy()
        out[f"km_{count}_{iters}_ids"] = ids.numpy()
    # constant input: every token identical (reference tests/test_cuda.py:161-169 shape of case)
    const = np.full((1, 1, 256, 128), 20.0, np.float16)
    cen, ids = rc.cluster(T(const), 4, 2)
    out["km_const_centres"], out["km_const_ids"] = cen.numpy(), ids.numpy()

    # ---- 5. incremental step ------------------------------------------------
    grp = mixture(rng, 1, 2, 64, clusters=6)
    prev = (rng.standard_normal((1, 2, 5, 128))).astype(np.float16)
    cfg = ResKVKernelConfig(num_clusters=4, max_clusters=6)
    out["inc_x"], out["inc_prev"] = grp, prev
    for value in (False, True):
        cen, ids = rc._incremental_cluster(T(grp), T(prev), cfg, value=value)
        out[f"inc_{int(value)}_centres"], out[f"inc_{int(value)}_ids"] = cen.numpy(), ids.numpy()
    full = (rng.standard_normal((1, 2, 6, 128))).astype(np.float16)
    out["inc_full_prev"] = full
    cen, ids = rc._incremental_cluster(T(grp), T(full), cfg)
    out["inc_full_centres"], out["inc_full_ids"] = cen.numpy(), ids.numpy()

    # ---- 6. linspace initial indices ---------------------------------------
    pairs = [(t_, c_) for t_ in (32, 33, 64, 100, 255, 1000, 8128, 16320, 65472) for c_ in (1, 2, 4, 31, 32, 64)
             if t_ >= c_]
    out["lin_pairs"] = np.array(pairs)
    out["lin_idx"] = np.concatenate([torch.linspace(0, t_ - 1, c_).long().numpy() for t_, c_ in pairs])

    np.savez_compressed(HERE / "reference_vectors.npz", **out)

    # ---- 7. plan resolution grid -------------------------------------------
    grid = []
    for sp, bits, layout, fusion, soft, batch in itertools.product(
            (0.5, 0.75), (2, 4, 16), ("auto", "unstructured", "tiled", "structured"),
            ("auto", "per_token", "deferred"), ("online", "fixed_shift"), (1, 2, 4, 8, 16, 32, 64)):
        settings = dict(sparsity=sp, bits=bits, layout=layout, centroid_fusion=fusion, softmax_mode=soft)
        try:
            plan = ResKVKernelConfig(**settings).resolve(batch).to_dict()
        except ValueError as e:
            plan = {"error": str(e)}
        grid.append({"settings": settings, "batch": batch, "plan": plan})
    (HERE / "plan_grid.json").write_text(json.dumps(grid, separators=(",", ":")))
    print("wrote", HERE / "reference_vectors.npz", (HERE / "reference_vectors.npz").stat().st_size, "bytes;",
          len(grid), "plan cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
