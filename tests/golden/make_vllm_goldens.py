"""Generates tests/golden/vllm_comparator.npz: outputs of vLLM's Triton block-fp8 fused-MoE pipeline
(the upstream of the SGLang pipeline the reference's correctness script compares against,
test/test_moe_correctness.py:77-110) on seeded cases of this repository's input generators.
Needs a CUDA device and the vllm package: `python tests/golden/make_vllm_goldens.py [--out FILE]`.
The fixture is committed, so the CPU tests can hold the oracle against results that this
repository's authors did not compute, without vLLM or a GPU at test time.

Stored per case: SHA-256 of the seeded inputs (so that a drifting generator is noticed), the
comparator's bf16 output (as raw uint16), vLLM's group-quantised activations / scales, and vLLM's
block schedule for block size 16.
"""
import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import moe_oracle as orc          # noqa: E402
from tests import vllm_comparator as vc      # noqa: E402

CASES = {
    # BASELINE config 0: E=8, K=512, I=128, M=16, top_k=2, seed 0
    "cfg0": lambda: orc.make_case(8, 512, 128, 16, 2, seed=0),
    # a two-slice shape with the shared expert and routed scaling
    "ds_small": lambda: orc.make_case(16, 1024, 256, 40, 5, seed=3, shared=True, scaling=2.5),
    # the reference's own input distribution (test_moe_correctness.py:49-67), duplicates inside a token included
    "refdist": lambda: orc.make_reference_style_case(32, 8, 512, 1024, 9),
}


def digest(case) -> str:
    h = hashlib.sha256()
    for name in ("x", "x_scale", "w", "w_scale", "w2", "w2_scale", "topk_ids", "topk_weights", "x_bf16"):
        t = getattr(case, name).contiguous()
        if t.dtype == torch.float8_e4m3fn:
            t = t.view(torch.uint8)
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        h.update(t.numpy().tobytes())
    return h.hexdigest()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "vllm_comparator.npz"))
    args = ap.parse_args()
    import vllm
    blob = {"vllm_version": np.array(vllm.__version__)}
    for name, make in CASES.items():
        case = make()
        out = vc.vllm_fused_moe(case)
        q, s = vc.vllm_group_quant(case.x_bf16)
        sid, eid, npp = vc.vllm_align(case.topk_ids, 16, case.num_experts)
        blob[f"{name}_sha256"] = np.array(digest(case))
        blob[f"{name}_out_bf16"] = out.view(torch.int16).numpy()
        blob[f"{name}_xq"] = q.view(torch.uint8).numpy()
        blob[f"{name}_xs"] = s.numpy()
        blob[f"{name}_sid"] = sid.numpy()
        blob[f"{name}_eid"] = eid.numpy()
        blob[f"{name}_npp"] = npp.numpy()
        ref = orc.run_oracle(case, 16)
        print(name, "rel-L2 oracle vs vLLM:", orc.rel_l2(ref, out), "max|d|", float((ref.float() - out.float()).abs().max()))
    np.savez_compressed(args.out, **blob)
    print("wrote", args.out)


if __name__ == "__main__":
    main()
