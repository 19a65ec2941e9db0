"""Generates the golden fixtures of this directory.  Run once, where a checkout of the reference
(Aleph-Alpha/Alpha-MoE) is at hand: `ALPHA_MOE_REFERENCE=<checkout> python make_reference_goldens.py`.
The fixtures are committed so that the tests never read the reference at run time.

  ref_interleave.npz     outputs of the reference's alpha_moe_python.utils.interleave_tensor
                         (imported from the reference) on fixed integer inputs, rep = 8 / 1 / 2
  ref_best_config.json   outputs of the reference's get_best_config on a table written by this script
  cfg0_oracle.npz        config 0 (E=8, K=512, I=128, M=16, top_k=2, block_m=16, seed 0): SHA-256 of the
                         seeded operator inputs, the block schedule, and the output of *this
                         repository's* oracle (both variants).  The reference pins no results for the
                         operator itself, so this file is a regression pin of the oracle and of the
                         input generator, not a reference result.
"""
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("ALPHA_MOE_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set ALPHA_MOE_REFERENCE to a checkout of the reference repository")


def load_reference_utils():
    spec = importlib.util.spec_from_file_location("ref_utils", os.path.join(REF, "alpha_moe_python", "utils.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def case_digest(case) -> str:
    """SHA-256 over the raw bytes of every operator input of a seeded case."""
    import hashlib
    h = hashlib.sha256()
    for name in ("x", "x_scale", "w", "w_scale", "w2", "w2_scale", "topk_ids", "topk_weights"):
        t = getattr(case, name).contiguous()
        if t.dtype == torch.float8_e4m3fn:
            t = t.view(torch.uint8)
        h.update(t.numpy().tobytes())
    return h.hexdigest()


def main():
    ref = load_reference_utils()
    # --- interleave_tensor
    a = torch.arange(2 * 32 * 3, dtype=torch.int32).reshape(2, 32, 3)
    b = torch.arange(3 * 256 * 2, dtype=torch.int32).reshape(3, 256, 2)
    s = torch.arange(2 * 4 * 5, dtype=torch.int32).reshape(2, 4, 5)
    np.savez_compressed(
        os.path.join(HERE, "ref_interleave.npz"),
        a=a.numpy(), a_rep8=ref.interleave_tensor(a, 8).numpy(), a_rep2=ref.interleave_tensor(a, 2).numpy(),
        b=b.numpy(), b_rep8=ref.interleave_tensor(b, 8).numpy(),
        s=s.numpy(), s_rep1=ref.interleave_tensor(s, 1).numpy())
    # --- get_best_config (nearest bucket, first wins on ties)
    table = {"1": {"block_m": 16, "block_n": 32, "warp_n": 8, "stages": 5},
             "8": {"block_m": 8, "block_n": 32, "warp_n": 8, "stages": 4},
             "64": {"block_m": 8, "block_n": 64, "warp_n": 4, "stages": 2},
             "1024": {"block_m": 32, "block_n": 64, "warp_n": 4, "stages": 2},
             "4096": {"block_m": 80, "block_n": 32, "warp_n": 8, "stages": 5}}
    tpath = os.path.join(HERE, "best_config_table.json")
    with open(tpath, "w") as f:
        json.dump(table, f)
    queries = [1, 2, 4, 5, 8, 36, 37, 64, 544, 545, 2560, 2561, 100000]
    got = {str(q): ref.get_best_config(tpath, q) for q in queries}
    with open(os.path.join(HERE, "ref_best_config.json"), "w") as f:
        json.dump(got, f, indent=1)
    # --- config 0, this repository's oracle
    from oracle import moe_oracle as orc
    case = orc.make_case(8, 512, 128, 16, 2, seed=0)
    sid, eid, npp = case.schedule(16)
    out_b = orc.run_oracle(case, 16, faithful=True, out_fp32=True)
    out_a = orc.run_oracle(case, 16, faithful=False, out_fp32=True)
    np.savez_compressed(
        os.path.join(HERE, "cfg0_oracle.npz"),
        inputs_sha256=np.array(case_digest(case)),
        topk_ids=case.topk_ids.numpy(), topk_weights=case.topk_weights.numpy(),
        sorted_token_ids=sid.numpy(), expert_ids=eid.numpy(), num_tokens_post_padded=npp.numpy(),
        out_faithful=out_b.numpy(), out_ideal=out_a.numpy())
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
