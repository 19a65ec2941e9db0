"""The knob search (counterpart of the reference's jit_moe.py) on a small shape: it must write a table in the
reference's format whose entries come from the searched tuples, `get_best_config` must read it, and the operator must
accept what it picked.  Both timing methods run: CUDA events and the reference's torch.profiler method."""
import json

import pytest
import torch

pytestmark = pytest.mark.gpu
KNOBS = ["16,32,8,3", "16,64,4,2", "64,64,4,2", "128,64,4,3"]


@pytest.mark.parametrize("timing", ["events", "kineto"])
def test_tuner_writes_a_valid_table(tmp_path, timing):
    from alpha_moe_b200 import tune
    from alpha_moe_b200.utils import get_best_config
    out = tmp_path / f"table_{timing}.json"
    table, report = tune.main(["--E", "16", "--N", "512", "--K", "1024", "--top-k", "4", "--batch-sizes", "4", "200",
                               "--routings", "1", "--iters", "2", "--knobs", *KNOBS, "--timing", timing,
                               "--out-file", str(out)])
    on_disk = json.loads(out.read_text())
    assert on_disk == table and set(table) == {"4", "200"}
    allowed = [tuple(int(v) for v in k.split(",")) for k in KNOBS]
    for m, conf in table.items():
        assert set(conf) == {"block_m", "block_n", "warp_n", "stages"}
        assert (conf["block_m"], conf["block_n"], conf["warp_n"], conf["stages"]) in allowed
        assert 0 < report[int(m)] < 1e5
    assert table["4"]["block_m"] == 16                      # blocks larger than the batch are pruned, except 16
    assert get_best_config(str(out), 150) == table["200"]   # nearest bucket
    # the operator accepts what was picked
    from oracle import moe_oracle as orc
    from tests.harness import check_close, run_capi
    case = orc.make_case(8, 512, 256, 40, 2, seed=3)
    c = table["200"]
    check_close(run_capi(case, c["block_m"], c["block_n"], c["warp_n"], c["stages"]), orc.run_oracle(case, c["block_m"]))


def test_tuner_rejects_malformed_knob_tuples():
    from alpha_moe_b200 import tune
    with pytest.raises(ValueError):
        tune.parse_knobs(["16,32,8"])
