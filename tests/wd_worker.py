"""Worker for the failure-detection tests: CPU ranks (gloo) with a watchdog; one rank misbehaves as told."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from surogate_b200.parallel.dist import init_distributed  # noqa: E402
from surogate_b200.parallel.watchdog import RemoteRankFailed, install  # noqa: E402


def main():
    a = json.loads(sys.argv[1])
    info = init_distributed(backend="gloo", timeout_s=a.get("pg_timeout_s", 20))
    wd = install(info.rank, info.world, heartbeat_s=0.2, stale_after_s=a.get("stale_after_s", 2.0), abort_after_s=a.get("abort_after_s", 5.0))
    out = {"rank": info.rank, "steps": 0}
    try:
        with wd.guard():
            for step in range(a.get("steps", 50)):
                wd.tick(step)
                wd.check()  # before the step's first collective
                if info.rank == a.get("bad_rank", 1) and step == a.get("fail_at", 3):
                    if a["mode"] == "raise":
                        raise ValueError("synthetic failure: bad batch at step %d" % step)
                    if a["mode"] == "exit":
                        os._exit(17)  # dies without a note, between steps, with no collective in flight
                t = torch.ones(4) * (info.rank + 1)
                dist.all_reduce(t)
                out["steps"] = step + 1
                time.sleep(0.25)
    except RemoteRankFailed as e:
        out["remote_failure"] = {"rank": e.rank, "reason": e.reason}
    except ValueError as e:
        out["own_failure"] = str(e)
    except RuntimeError as e:  # the collective itself ended with an error (peer gone): also a clean, bounded exit
        out["collective_error"] = str(e)[:200]
    print("RESULT " + json.dumps(out), flush=True)
    wd.stop()
    os._exit(0)  # skip process-group teardown: the peer may be gone


if __name__ == "__main__":
    main()
