"""Runs the reference's GLM engine, unmodified (c/colibri.c built by `make -C oracle dropin` with
this repository's library where c/backend_cuda.o stands), on a converted checkpoint directory:
once on the CPU and then with COLI_CUDA=1 in the call sequences its moe() has for a GPU
backend (c/colibri.c:4819-4921 synchronous groups, :4467/:4791 COLI_GROUP_ASYNC, CUDA_DENSE
for the resident dense tensors), and prints, per mode, the greedy token line, the
teacher-forced agreement and the REPLAY throughput / P0-EXEC lines
(the replay of c/tools/benchmark_cuda_fixture.py:76-101).

    python oracle/dropin_demo.py --snap <dir made by c/tools/make_glm_bench_model.py + convert_fp8_to_int4.py>

TEST INFRASTRUCTURE: nothing in the library or bench.py imports this."""
import argparse
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENGINE = os.path.join(ROOT, "oracle", "_ref", "colibri_b200")

MODES = [
    ("cpu", {}),
    ("cuda experts, synchronous groups", {"COLI_CUDA": "1", "COLI_GPUS": "0", "PIN": "@stats", "PIN_GB": "1", "CUDA_EXPERT_GB": "2"}),
    ("cuda experts, COLI_GROUP_ASYNC=1", {"COLI_CUDA": "1", "COLI_GPUS": "0", "PIN": "@stats", "PIN_GB": "1", "CUDA_EXPERT_GB": "2",
                                          "COLI_GROUP_ASYNC": "1"}),
    ("cuda experts + CUDA_DENSE=1", {"COLI_CUDA": "1", "COLI_GPUS": "0", "PIN": "@stats", "PIN_GB": "1", "CUDA_EXPERT_GB": "2",
                                     "CUDA_DENSE": "1"}),
]


def run(snap, extra, mode_env):
    env = dict(os.environ)
    for k in ("COLI_CUDA", "COLI_GPU", "COLI_GPUS", "CUDA_EXPERT_GB", "PIN", "PIN_GB", "STATS", "TF", "REPLAY", "CUDA_DENSE",
              "COLI_GROUP_ASYNC"):
        env.pop(k, None)
    env.update(SNAP=snap, REF=os.path.join(snap, "ref_glm.json"), DRAFT="0", COLI_NO_OMP_TUNE="1")
    env.update({k: (os.path.join(snap, "bench_stats.txt") if v == "@stats" else v) for k, v in mode_env.items()})
    env.update(extra)
    p = subprocess.run([ENGINE, "4", "4", "4"], env=env, capture_output=True, text=True, timeout=600)
    return p.returncode, p.stdout, p.stderr


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--snap", required=True)
    args = ap.parse_args()
    snap = os.path.abspath(args.snap)
    if not os.path.exists(os.path.join(snap, "bench_stats.txt")):
        run(snap, {"REPLAY": "1", "STATS": os.path.join(snap, "bench_stats.txt")}, {})     # the usage histogram PIN= reads
    base_tokens = None
    for name, menv in MODES:
        print(f"== {name}")
        rc, out, err = run(snap, {}, menv)
        tok = re.search(r"GLM C engine\s*:\s*([0-9 ]+)", out)
        tokens = tok.group(1).split() if tok else None
        if base_tokens is None:
            base_tokens = tokens
        tier = re.search(r"CUDA expert tier:.*", out)
        print(f"   greedy tokens : {' '.join(tokens) if tokens else 'none (rc %d)' % rc}"
              f"{'' if tokens is None or tokens == base_tokens else '   <-- differs from the CPU run'}")
        if tier:
            print("   " + tier.group(0))
        rc, out, err = run(snap, {"TF": "1"}, menv)
        tf = re.search(r"PREFILL \(teacher-forcing\).*", out)
        print("   " + (tf.group(0) if tf else f"TF run failed (rc {rc})"))
        rc, out, err = run(snap, {"REPLAY": "1", "PROF": "1"}, menv)
        for pat in (r"REPLAY decode:.*", r"P0-EXEC:.*"):
            m = re.search(pat, out)
            print("   " + (m.group(0) if m else f"{pat} missing (rc {rc})"))
        notes = [l for l in (out + err).splitlines() if "[CUDA]" in l][:6]
        for l in notes:
            print("   " + l)


if __name__ == "__main__":
    main()
