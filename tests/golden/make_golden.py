"""Generates tests/golden/reference_b200.pt: outputs of the reference project's own CUDA kernels
(oracle/_ref/librisa_ref.so, built by oracle/build_ref.sh from the unmodified reference sources)
on a B200, for small seeded inputs.  Run on a GPU box:

    python tests/golden/make_golden.py [output path]

The inputs are regenerated from the seeds by the tests (CPU generator), so only results are stored.
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import ref_gpu  # noqa: E402

CASES = [
    # seed, (b, hq, hkv, lq, lk, d), cta_k, affine, anchor, theta
    (11, (1, 2, 1, 137, 263, 128), 64, False, False, 0.9),
    (12, (1, 4, 2, 200, 1153, 128), 128, True, True, 0.99),
    (13, (2, 2, 2, 70, 300, 64), 64, True, False, 0.5),
    (14, (1, 2, 1, 130, 1100, 256), 128, False, True, 0.99),
]


def main(out_path):
    cases = []
    for seed, shape, cta_k, affine, anchor, theta in CASES:
        b, hq, hkv, lq, lk, d = shape
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(b, hq, lq, d, generator=g).bfloat16()
        k = torch.randn(b, hkv, lk, d, generator=g).bfloat16()
        v = torch.randn(b, hkv, lk, d, generator=g).bfloat16()
        if anchor:
            k = (k.float() * 0.1 + 4).bfloat16()
        pk = ref_gpu.prequantize(q.cuda(), k.cuda(), v.cuda(), cta_k=cta_k, midpoint_affine=affine)
        r = ref_gpu.attention(pk, sm_scale=d ** -0.5, capture=True, want_lse=True)
        n_q, n_k = -(-lq // 128), -(-lk // cta_k)
        masses = r["workspace"][: b * hq * n_q * n_k].view(-1, n_k).clone()
        ro, bi, measured = ref_gpu.select_retained_mass(masses, theta)
        torch.cuda.synchronize()
        cases.append({
            "seed": seed, "shape": shape, "cta_k": cta_k, "affine": affine, "anchor": anchor,
            "theta": theta, "anchors": pk["anchors"].cpu(), "q": pk["q"].cpu(), "k": pk["k"].cpu(),
            "v": pk["v"].cpu(), "q_scale": pk["q_scale"].cpu(), "k_scale": pk["k_scale"].cpu(),
            "v_scale": pk["v_scale"].cpu(), "v_center": pk["v_center"].cpu(),
            "out": r["out"].cpu(), "lse": r["lse"].cpu(), "masses": masses.cpu(),
            "row_offsets": ro.cpu(), "block_indices": bi.cpu(), "measured_mass": measured,
        })
    torch.save({"gpu": torch.cuda.get_device_name(0), "cases": cases}, out_path)
    print("wrote", out_path)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else str(Path(__file__).with_name("reference_b200.pt")))
