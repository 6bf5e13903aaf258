"""Worker for the pipeline-parallel SFT test: runs the SFT loop with ``parallelism: dispatch_pp`` under torchrun (gloo, CPU)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from surogate_b200.config.sft_config import SFTConfig  # noqa: E402
from surogate_b200.train.sft import run_training  # noqa: E402

if __name__ == "__main__":
    r = run_training(SFTConfig.from_dict(json.loads(sys.argv[1])))
    if int(os.environ.get("RANK", "0")) == 0:
        print("RESULT " + json.dumps({"steps": r["steps"], "losses": r["losses"], "final": r["final"]}), flush=True)
