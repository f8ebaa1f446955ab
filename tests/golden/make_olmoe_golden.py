"""Pins the OLMoE decode harness (colibri_b200/olmoe_harness.py) and the oracle's softmax
top-K MoE against the reference engine itself.

Run in a container that has the reference checkout:
    python tests/golden/make_olmoe_golden.py
It builds the unmodified engine (c/olmoe.c -> oracle/_ref/olmoe_ref, recipe in
oracle/Makefile), writes a small synthetic snapshot in the engine's own container format
(config.json + model.safetensors: dense f32 tensors, per-expert merged int8 blob
`gate|up|down` + `[I+I+D]` f32 scales, c/olmoe.c:413-438), runs the engine on a seeded
prompt with IDOT=0 (the f32 matvec, c/olmoe.c:207-236) and stores the token ids of its
`C engine :` line (c/olmoe.c:1404-1407) in tests/golden/olmoe_tokens.json together with
the seeds that regenerate the weights. tests/test_olmoe_pin.py then requires the harness,
with the CPU oracle as its MoE, to decode the same ids.
"""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from colibri_b200 import workloads as W  # noqa: E402
from colibri_b200.olmoe_harness import OlmoeModel  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
ENGINE = os.path.join(ROOT, "oracle", "_ref", "olmoe_ref")

CASES = [
    dict(name="tiny_k4", D=256, H=2, hd=128, layers=3, E=16, K=4, I=128, vocab=512, norm_topk=0,
         seed=11, prompt_len=8, n_new=24),
    dict(name="tiny_k8_norm", D=256, H=2, hd=128, layers=2, E=64, K=8, I=128, vocab=384, norm_topk=1,
         seed=12, prompt_len=5, n_new=16),
]


def case_weights(c):
    """-> (OlmoeModel, [HostLayerWeights per layer]) regenerated from the case's seed."""
    m = OlmoeModel(c["D"], c["H"], c["hd"], c["layers"], c["vocab"], 10000.0, 1e-5, c["seed"], norm_jitter=0.1)
    cfg = dict(D=c["D"], I=c["I"], E=c["E"], K=c["K"], gating=0, norm_topk=c["norm_topk"], shared=False,
               fmt=1, gs=0)
    layers = [W.HostLayerWeights(cfg, c["seed"] * 31 + li, with_router=True) for li in range(c["layers"])]
    return m, cfg, layers


def case_prompt(c):
    return np.random.default_rng(c["seed"] + 1000).integers(0, c["vocab"], size=c["prompt_len"]).tolist()


def write_snapshot(c, d):
    from safetensors.numpy import save_file
    m, cfg, layers = case_weights(c)
    t = {"model.embed_tokens.weight": m.embed, "lm_head.weight": m.lm_head, "model.norm.weight": m.final_norm}
    for li, (dl, ml) in enumerate(zip(m.layers, layers)):
        p = f"model.layers.{li}."
        t[p + "input_layernorm.weight"] = dl["in_ln"]
        t[p + "post_attention_layernorm.weight"] = dl["post_ln"]
        for k in "qkvo":
            t[p + f"self_attn.{k}_proj.weight"] = dl[k]
        t[p + "self_attn.q_norm.weight"] = dl["qn"]
        t[p + "self_attn.k_norm.weight"] = dl["kn"]
        t[p + "mlp.gate.weight"] = ml.router_w
        for e in range(c["E"]):
            g, u, dn = ml.gate[e], ml.up[e], ml.down[e]
            t[p + f"mlp.experts.{e}.merged_weight"] = np.concatenate(
                [g.w.reshape(-1), u.w.reshape(-1), dn.w.reshape(-1)]).astype(np.int8)
            t[p + f"mlp.experts.{e}.qs"] = np.concatenate([g.s, u.s, dn.s]).astype(np.float32)
    save_file({k: np.ascontiguousarray(v) for k, v in t.items()}, os.path.join(d, "model.safetensors"))
    json.dump(dict(hidden_size=c["D"], num_hidden_layers=c["layers"], num_attention_heads=c["H"],
                   num_key_value_heads=c["H"], num_experts=c["E"], num_experts_per_tok=c["K"],
                   intermediate_size=c["I"], vocab_size=c["vocab"], rope_theta=10000.0, rms_norm_eps=1e-5,
                   norm_topk_prob=bool(c["norm_topk"])), open(os.path.join(d, "config.json"), "w"))
    prompt = case_prompt(c)
    json.dump(dict(prompt_ids=prompt, full_ids=prompt + [0] * c["n_new"]), open(os.path.join(d, "ref.json"), "w"))


def run_engine(c):
    """Token ids the unmodified engine decodes for the case."""
    with tempfile.TemporaryDirectory() as d:
        write_snapshot(c, d)
        env = dict(os.environ, SNAP=d, IDOT="0", OMP_NUM_THREADS="1")
        out = subprocess.run([ENGINE, "16", "8", os.path.join(d, "ref.json")], env=env, capture_output=True,
                             text=True, check=True).stdout
    line = [l for l in out.splitlines() if l.startswith("C engine :")][0]
    return [int(v) for v in line[len("C engine :"):].split()]


def main():
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "olmoe"])
    res = {}
    for c in CASES:
        res[c["name"]] = dict(case=c, prompt=case_prompt(c), tokens=run_engine(c))
        print(c["name"], res[c["name"]]["tokens"])
    json.dump(res, open(os.path.join(HERE, "olmoe_tokens.json"), "w"), indent=1)


if __name__ == "__main__":
    main()
