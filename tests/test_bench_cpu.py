"""bench.py pieces that run without a GPU: the reference (CPU) arm, its behaviour under a
multi-rank launch, and the cross-rank reduction over a world_size-2 gloo group."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _run(args, env_extra=None, timeout=600):
    env = dict(os.environ)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, capture_output=True,
                          text=True, timeout=timeout, env=env, cwd=ROOT)


def test_reference_arm_prints_the_contract_line():
    r = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"])
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["value"] == line["value"]
    assert line["value"] > 0


def test_reference_arm_under_a_multi_rank_launch():
    # rank 0 alone measures and prints; the other ranks exit 0 without work
    r1 = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
              {"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert r1.returncode == 0 and r1.stdout.strip() == ""
    r0 = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
              {"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "2", "OMP_NUM_THREADS": "1"})
    assert r0.returncode == 0
    line = json.loads(r0.stdout.strip().splitlines()[-1])
    assert line["n_gpus"] == 2
    # torchrun pins OMP_NUM_THREADS to 1; the arm must still use the host's cores
    assert line["cpu_baseline"]["cores"] == (os.cpu_count() or 1)


def test_max_over_ranks_and_shards_with_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys, json
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        import bench
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        ms = bench.max_over_ranks(10.0 + 5.0 * rank, dist, "cpu")   # rank 1 is the slow one
        first, count = bench.shard_of(rank, world, bench.GLOBAL_BATCH)               # strong: the batch is split
        wfirst, wcount = bench.shard_of(rank, world, bench.B_PER_GPU, "weak")        # weak: everyone runs it all
        print(json.dumps({{"rank": rank, "ms": ms, "first": first, "count": count, "wfirst": wfirst, "wcount": wcount}}))
        dist.destroy_process_group()
    """))
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT="29531")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1][-500:] for o in outs]
    res = sorted((json.loads(o[0].strip().splitlines()[-1]) for o in outs), key=lambda d: d["rank"])
    assert [d["ms"] for d in res] == [15.0, 15.0]          # both ranks see the slowest rank's time
    assert [d["first"] for d in res] == [0, 128] and all(d["count"] == 128 for d in res)
    assert [d["wfirst"] for d in res] == [0, 256] and all(d["wcount"] == 256 for d in res)


def test_strong_shards_cover_the_global_batch_exactly():
    import bench
    for world in (1, 2, 3, 4, 8):
        shards = [bench.shard_of(r, world, 256) for r in range(world)]
        assert shards[0][0] == 0 and sum(c for _, c in shards) == 256
        for (f0, c0), (f1, _) in zip(shards, shards[1:]):
            assert f0 + c0 == f1
