"""Host-side fault injection under gloo (no GPU involved): rank 1 leaves between steps.
  (a) the survivor learns of it through the heartbeat store before its next collective and stops cleanly;
  (b) without the heartbeat, the next collective ends with an error after the short process-group timeout."""
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindspeed_mm_b200.runtime.tools import PeerHeartbeat  # noqa: E402


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=4))
    store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]) + 1, world, rank == 0,
                          timeout=datetime.timedelta(seconds=20))
    hb = PeerHeartbeat(store, rank, world, timeout_s=30.0)
    x = torch.ones(4)
    for it in range(3):
        if mode == "heartbeat":
            bad = hb.failed_peers()
            if bad:
                print(f"rank {rank} stops before step {it}: peers {bad}", flush=True)
                print("dist_failure_check detected=heartbeat ok=True", flush=True)
                os._exit(0)
        if it == 1 and rank == 1:
            hb.leave("injected fault")           # between steps: nothing of this rank is in flight
            time.sleep(0.5)
            os._exit(0)
        try:
            dist.all_reduce(x)
        except Exception as e:  # noqa: BLE001
            print(f"rank {rank} collective failed at step {it}: {type(e).__name__}", flush=True)
            print("dist_failure_check detected=timeout ok=True", flush=True)
            os._exit(0)
        hb.beat(it)
        time.sleep(1.0 if rank == 0 else 0.0)     # give the leaving rank's note time to land
    print("dist_failure_check ok=False (no failure seen)", flush=True)
    os._exit(1)


if __name__ == "__main__":
    main()
