"""Records outputs of the reference's own CUDA code as golden fixtures.

Run on a machine with a CUDA device where the reference checkout is importable
(its three extension families are JIT-built by ``torch.utils.cpp_extension``
on first use; set ``RESKV_CACHE_DIR`` to reuse an earlier build):

    python tests/golden/make_golden_gpu.py /path/to/ResKV [output.npz]

All inputs are generated on the CPU from fixed seeds and stored next to the
outputs, so the consumers never depend on a device generator.  Recorded:

* the three packers that exist only as CUDA kernels in the reference
  (``reskv/csrc/compression.cu:57-147`` tiled and 4:16 FP16, ``:153-239`` 1-of-4
  INT4, ``:244-383`` INT4 / INT2 with nnz 32 and 64), called through
  ``reskv.compression._encode`` on a cluster-mixture input with outlier channels
  plus rows of ties, zeros, extremes and subnormals;
* the torch encoder of the unstructured FP16 layout run on the device
  (``reskv/compression.py:75-89``);
* ``cluster(value=True)`` (``reskv/compression.py:38-53``, the FP16 ``bmm``
  path that only runs on CUDA), ``cluster(value=False)`` on the device, and
  ``_incremental_cluster`` for both flavours;
* ``compress`` + ``attention`` for the eleven (bits, sparsity, layout, fusion)
  plans of the reference's ``tests/test_cuda.py:12-24``, with and without a
  recent window, next to ``reference_attention`` of the same cache;
* one full-size quantised case (16 320 compressed tokens, theta 1e6, INT4 and
  INT2): inputs come from ``reskv_b200.synthetic.mixture`` with a stored seed
  and are *not* stored; stored are the cluster tables, SHA-256 digests of the
  reference's packed words / scales and its attention outputs.

Consumers: ``tests/test_oracle_gpu_golden.py`` (CPU restatement against these
vectors) and ``tests/test_gpu_reference_vectors.py`` (this library against them).
"""

from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent

CASES = [
    (16, 0.5, "tiled", "per_token"),
    (16, 0.5, "unstructured", "deferred"),
    (16, 0.75, "unstructured", "deferred"),
    (16, 0.75, "structured", "per_token"),
    (16, 0.75, "structured", "deferred"),
    (4, 0.5, "unstructured", "per_token"),
    (4, 0.75, "unstructured", "per_token"),
    (4, 0.75, "structured", "per_token"),
    (4, 0.75, "structured", "deferred"),
    (2, 0.5, "unstructured", "per_token"),
    (2, 0.75, "unstructured", "per_token"),
]
PACKER_PLANS = [("tiled", 16, 64), ("structured", 16, 32), ("structured", 4, 32), ("unstructured", 4, 32),
                ("unstructured", 4, 64), ("unstructured", 2, 32), ("unstructured", 2, 64)]


def case_tag(bits, sparsity, layout, fusion):
    return f"{layout}_{bits}_{int(128 * (1 - sparsity))}_{fusion}"


def mixture_np(rng, b, h, t, clusters=8, sigma=0.3):
    centres = rng.standard_normal((b, h, clusters, 128)).astype(np.float32)
    which = rng.integers(0, clusters, (b, h, t))
    x = np.take_along_axis(centres, np.broadcast_to(which[..., None], (b, h, t, 128)), axis=2)
    x = x + sigma * rng.standard_normal((b, h, t, 128)).astype(np.float32)
    x = x * np.exp(rng.standard_normal((b, h, 1, 128))).astype(np.float32)
    return x.astype(np.float16)


def special_rows():
    """Ties, zeros, extremes, subnormals, near-boundary quotients."""
    rows = [np.ones(128), np.zeros(128), -np.ones(128) * 3, np.arange(1, 129), -np.arange(1, 129)[::-1],
            np.tile([5, 5, -5, 5, 1, 1, 1, 1], 16), np.full(128, 60000.0), np.full(128, 6e-8),
            np.tile([6e-8, 0, -6e-8, 1.2e-7], 32), np.linspace(-7, 7, 128), np.linspace(-3.5, 3.5, 128) * 1.0009765625,
            np.concatenate([np.full(64, 2.5), np.full(64, -1.5)])]
    return np.stack(rows).astype(np.float16)


def digest(t: torch.Tensor) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(t.detach().cpu().contiguous().numpy().tobytes()).digest(), np.uint8).copy()


def main(ref_root: str, out_path: Path):
    sys.path.insert(0, str(ROOT))   # reskv_b200.synthetic (the full-size inputs)
    sys.path.insert(0, ref_root)    # first: `reskv` must be the reference, not this repository's alias package
    import reskv.compression as rc
    if Path(rc.__file__).resolve().is_relative_to(ROOT / "reskv"):
        sys.exit("`reskv` resolved to this repository's alias package; pass the path of the reference checkout")
    import reskv.reference as rr
    from reskv import ResKVKernelConfig, attention, compress
    from reskv.config import KernelPlan

    dev = "cuda"
    out = {}
    rng = np.random.default_rng(20241125)
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    N = lambda t: t.detach().cpu().numpy()  # noqa: E731

    def plan_for(layout, bits, nnz):
        fusion = {"unstructured": "deferred" if bits == 16 else "per_token", "tiled": "per_token",
                  "structured": "deferred"}[layout]
        return KernelPlan(layout, fusion, bits, nnz, 4, 0)

    # ---- 1. the CUDA-only packers ---------------------------------------------
    b, h, c = 1, 2, 32
    spec = special_rows()
    body = mixture_np(rng, b, h, 180)
    x = np.concatenate([body, np.broadcast_to(spec[None, None], (b, h, *spec.shape))], axis=2)
    t = x.shape[2]
    cen = (rng.standard_normal((b, h, c, 128)) * 0.5).astype(np.float16)
    ids = rng.integers(0, c, (b, h, t)).astype(np.int32)
    cen[:, :, 0] = 0          # the special rows are encoded against an all-zero and a constant centre
    cen[:, :, 1] = 0.5
    ids[:, :, 180:] = np.arange(spec.shape[0]) % 2
    out.update(pk_x=x, pk_cen=cen, pk_ids=ids)
    for layout, bits, nnz in PACKER_PLANS:
        ct = rc._encode(T(x), T(cen), T(ids), plan_for(layout, bits, nnz))
        key = f"pk_{layout}_{bits}_{nnz}"
        out[key + "_payload"] = N(ct.payload)
        if ct.metadata is not None:
            out[key + "_meta"] = N(ct.metadata)
        if ct.scale is not None:
            out[key + "_scale"] = N(ct.scale)
        out[key + "_dense"] = N(rr.reconstruct(ct))
    for nnz in (32, 64):
        for value in (False, True):
            ct = rc._encode(T(x), T(cen), T(ids), plan_for("unstructured", 16, nnz), value=value)
            key = f"pk_unstructured_16_{nnz}_{'v' if value else 'k'}"
            out[key + "_payload"], out[key + "_meta"] = N(ct.payload), N(ct.metadata)

    # ---- 2. clustering on the device ------------------------------------------
    xk = mixture_np(rng, 1, 2, 512, clusters=6)
    out["km_x"] = xk
    for value in (False, True):
        for count, iters in ((8, 1), (8, 4), (32, 3), (32, 10)):
            cen_o, ids_o = rc.cluster(T(xk), count, iters, value=value)
            key = f"km_{int(value)}_{count}_{iters}"
            out[key + "_centres"], out[key + "_ids"] = N(cen_o), N(ids_o)
    const = np.full((1, 1, 8192, 128), 20.0, np.float16)
    for count in (1, 32):
        cen_o, ids_o = rc.cluster(T(const), count=count, iterations=2, value=True)
        out[f"km_const_{count}_centres"], out[f"km_const_{count}_ids"] = N(cen_o), N(ids_o)
    grp = mixture_np(rng, 1, 2, 64, clusters=6)
    prev = rng.standard_normal((1, 2, 5, 128)).astype(np.float16)
    cfg = ResKVKernelConfig(num_clusters=4, max_clusters=6)
    out["inc_x"], out["inc_prev"] = grp, prev
    for value in (False, True):
        cen_o, ids_o = rc._incremental_cluster(T(grp), T(prev), cfg, value=value)
        out[f"inc_{int(value)}_centres"], out[f"inc_{int(value)}_ids"] = N(cen_o), N(ids_o)

    # ---- 3. the eleven plans of the reference's attention test -----------------
    bb, hh, tt = 1, 2, 256
    k = (rng.standard_normal((bb, hh, tt, 128)) * 0.5).astype(np.float16)
    v = (rng.standard_normal((bb, hh, tt, 128)) * 0.5).astype(np.float16)
    q = (rng.standard_normal((bb, hh * 4, 1, 128)) * 0.5).astype(np.float16)
    kc = (rng.standard_normal((bb, hh, 32, 128)) * 0.1).astype(np.float16)
    vc = (rng.standard_normal((bb, hh, 32, 128)) * 0.1).astype(np.float16)
    ki = rng.integers(0, 32, (bb, hh, tt)).astype(np.int32)
    vi = rng.integers(0, 32, (bb, hh, tt)).astype(np.int32)
    kr = (rng.standard_normal((bb, hh, 32, 128)) * 0.5).astype(np.float16)
    vr = (rng.standard_normal((bb, hh, 32, 128)) * 0.5).astype(np.float16)
    freq = (500000.0 ** (-torch.arange(64).float() / 64) / torch.linspace(1, 8, 64)).numpy()
    out.update(at_k=k, at_v=v, at_q=q, at_kc=kc, at_vc=vc, at_ki=ki, at_vi=vi, at_kr=kr, at_vr=vr, at_freq=freq)
    qr = rr.rotate(T(q), torch.tensor([288], device=dev), T(freq)).half()
    out["at_qr"] = N(qr)
    for bits, sparsity, layout, fusion in CASES:
        cfg = ResKVKernelConfig(bits=bits, sparsity=sparsity, layout=layout, centroid_fusion=fusion)
        cache = compress(T(k), T(v), cfg, clustering=((T(kc), T(ki)), (T(vc), T(vi))))
        tag = "at_" + case_tag(bits, sparsity, layout, fusion)
        for side, ct in (("k", cache.key), ("v", cache.value)):
            out[f"{tag}_{side}_payload"] = N(ct.payload)
            if ct.metadata is not None:
                out[f"{tag}_{side}_meta"] = N(ct.metadata)
            if ct.scale is not None:
                out[f"{tag}_{side}_scale"] = N(ct.scale)
        out[tag + "_out"] = N(attention(T(q), cache, position=288, inv_freq=T(freq)))
        out[tag + "_ref"] = N(rr.reference_attention(T(q), cache, position=288, inv_freq=T(freq)))
        recent = (qr, T(kr), T(vr))
        out[tag + "_out_recent"] = N(attention(T(q), cache, position=288, inv_freq=T(freq), recent=recent))
        out[tag + "_ref_recent"] = N(rr.reference_attention(T(q), cache, position=288, inv_freq=T(freq), recent=recent))

    # ---- 4. full-size quantised case: 16 320 tokens, theta 1e6 -----------------
    from reskv_b200.synthetic import gaussian, mixture

    fb, fh, ft, seed = 1, 2, 16320, 77
    fk = mixture(fb, fh, ft, seed=seed)
    fv = mixture(fb, fh, ft, seed=seed + 1)
    fq = gaussian(fb, fh * 4, 1, 128, seed=seed + 2)
    out["fs_shape"] = np.array([fb, fh, ft, seed])
    out["fs_k_digest"], out["fs_v_digest"], out["fs_q"] = digest(fk), digest(fv), N(fq)
    fkc, fki = rc.cluster(fk.to(dev), 32, 15)
    fvc, fvi = rc.cluster(fv.to(dev), 32, 15, value=True)
    out.update(fs_kc=N(fkc), fs_ki=N(fki).astype(np.int8), fs_vc=N(fvc), fs_vi=N(fvi).astype(np.int8))
    inv = (1e6 ** (-torch.arange(64).float() / 64)).to(dev)
    out["fs_freq"] = N(inv)
    for bits in (4, 2):
        cfg = ResKVKernelConfig(bits=bits, sparsity=0.5, layout="unstructured")
        cache = compress(fk.to(dev), fv.to(dev), cfg, clustering=((fkc, fki), (fvc, fvi)))
        tag = f"fs_int{bits}"
        out[tag + "_k_payload_digest"], out[tag + "_k_scale_digest"] = digest(cache.key.payload), digest(cache.key.scale)
        out[tag + "_v_payload_digest"], out[tag + "_v_scale_digest"] = digest(cache.value.payload), digest(cache.value.scale)
        out[tag + "_out"] = N(attention(fq.to(dev), cache, position=16384, inv_freq=inv))
        out[tag + "_ref"] = N(rr.reference_attention(fq.to(dev), cache, position=16384, inv_freq=inv))
    cfg = ResKVKernelConfig(bits=16, sparsity=0.75, layout="unstructured")
    cache = compress(fk.to(dev), fv.to(dev), cfg, clustering=((fkc, fki), (fvc, fvi)))
    out["fs_fp16_out"] = N(attention(fq.to(dev), cache, position=16384))
    out["fs_fp16_ref"] = N(rr.reference_attention(fq.to(dev), cache, position=16384))

    out["torch_version"] = np.array(torch.__version__)
    out["device_name"] = np.array(torch.cuda.get_device_name(0))
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, out_path.stat().st_size, "bytes,", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit("usage: python make_golden_gpu.py <path of the reference checkout> [output.npz]")
    main(sys.argv[1], Path(sys.argv[2]) if len(sys.argv) == 3 else HERE / "reference_gpu_vectors.npz")
