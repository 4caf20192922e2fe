"""Worker of test_multi_process.py: one rank of a world_size-2 gloo job exercising the bench's
multi-GPU host logic (shard planning, barrier, max-over-ranks) without a GPU."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bench  # noqa: E402


def main():
    d = bench.Dist("gloo")
    args = argparse.Namespace(workload="cfg5", global_batch=0, dequant="cached")
    cfg = bench.workload_config(args, d.world)
    assert cfg["global_batch"] == 1024 and cfg["per_gpu"] == 1024 // d.world and cfg["scaling"] == "strong"
    cfg4 = bench.workload_config(argparse.Namespace(workload="cfg4", global_batch=0, dequant="cached"), d.world)
    assert cfg4["per_gpu"] == 64 and cfg4["global_batch"] == 64 * d.world and cfg4["scaling"] == "weak"
    d.barrier()
    # the slowest rank defines the step time
    slowest = d.max(10.0 + d.rank)
    assert slowest == 10.0 + d.world - 1, slowest
    d.barrier()
    if d.rank == 0:
        print(f"ok world={d.world} per_gpu={cfg['per_gpu']}")
    d.close()


if __name__ == "__main__":
    main()
