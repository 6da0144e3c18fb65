"""Worker of the rank-loss test: the last rank leaves between two steps, the others notice on the host.

Rules the scenario follows: the leaving rank has no kernel or collective in flight (device synchronised, peers
past the step's last flag barrier); the survivors learn of the loss from the heartbeat store *before* their next
launch and launch nothing afterwards; in-switch reductions are off and the kernels use plain peer stores.
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["report", "silent"], default="report")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dist.init_process_group("gloo")
    from retinags_b200.bench_session import BenchSession
    from retinags_b200.parallel.watchdog import PeerFailure, Watchdog

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, is_master=rank == 0, wait_for_workers=True)
    dog = Watchdog(store, rank, world, interval=0.2, timeout=2.0).start()
    sess = BenchSession(dev, rank, world, transport="peer" if cuda else "nccl", n_gaussians=60000, width=320, height=208,
                        batch=2, n_views=4, gt_gaussians=20000, seed=2, sh_degree=3, grid=(64, 64, 1))
    for it in range(2):
        dog.check()
        sess.step_e2e(it)
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()  # every rank is between steps, nothing of the last step is in flight
    if cuda:
        torch.cuda.synchronize()
    if rank == world - 1:
        if a.mode == "report":
            dog.report_failure("injected: rank leaves between steps")
        dog.stop()
        print(f"rank {rank} leaves", flush=True)
        os._exit(0)  # no destructor launches anything
    deadline = time.monotonic() + 20.0
    detected = None
    while time.monotonic() < deadline:
        try:
            dog.check()  # the survivor polls the host-side state; it launches no kernel while it waits
        except PeerFailure as exc:
            detected = str(exc)
            break
        time.sleep(0.1)
    if detected is None:
        print("rank loss was not detected", flush=True)
        os._exit(1)
    if cuda:
        torch.cuda.synchronize()  # the context is still usable
        assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    print(f"RANK_LOSS_DETECTED rank {rank}: {detected}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
