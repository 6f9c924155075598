"""Generates tests/golden/*.npz by running the REFERENCE's own PyTorch path on seeded inputs.

Run where the reference checkout is available (default: a directory `reference` next to this repository; override
with REFERENCE_DIR):

    python tests/golden/make_golden.py

For each case the inputs come from fused_moe_b200.synth (bit-reproducible on any machine), the outputs from
solution/cuda/binding.py: ``_ds_routing_impl`` (binding.py:38-61) and ``kernel`` (binding.py:96-185) run on CPU with a
float32 destination so the un-rounded sums are kept.  Two module globals of binding.py are adjusted, nothing else:
``ds_routing`` is pointed at the un-compiled ``_ds_routing_impl`` (the file wraps it in torch.compile), and ``E_LOCAL``
is set to the case's expert count (the file hard-codes 32).  torch.topk(sorted=False) leaves the order of the eight
experts unspecified, so indices and weights are stored sorted by expert id per token.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from fused_moe_b200 import synth  # noqa: E402

REFERENCE_DIR = Path(os.environ.get("REFERENCE_DIR", str(HERE.parent.parent.parent / "reference")))

# name -> dict(T, E_local, offset, seed, skew, full[, heavy])   full=False: routing only (no expert weights needed);
# heavy=True: heavy-tailed activations (synth.make_inputs(heavy_tail=True))
CASES = {
    "config0_t7_e32": dict(T=7, E_local=32, offset=0, seed=0, skew=False, full=True),
    "t1_e32": dict(T=1, E_local=32, offset=96, seed=5, skew=False, full=True),
    "t33_e8_off60": dict(T=33, E_local=8, offset=60, seed=3, skew=False, full=True),
    "t40_e3_off253_skew": dict(T=40, E_local=3, offset=253, seed=13, skew=True, full=True),
    "t3_e2_none_local": dict(T=3, E_local=2, offset=100, seed=21, skew=False, full=True),
    "t12_e8_off16_heavy_tail": dict(T=12, E_local=8, offset=16, seed=34, skew=False, full=True, heavy=True),
    "route_t4096_skew": dict(T=4096, E_local=32, offset=0, seed=7, skew=True, full=False),
    "route_t1000": dict(T=1000, E_local=32, offset=0, seed=8, skew=False, full=False),
}


def load_binding():
    path = REFERENCE_DIR / "solution" / "cuda" / "binding.py"
    spec = importlib.util.spec_from_file_location("reference_binding", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.ds_routing = mod._ds_routing_impl
    return mod


def sorted_routing(idx: torch.Tensor, w: torch.Tensor):
    order = idx.argsort(dim=1)
    return torch.gather(idx, 1, order), torch.gather(w, 1, order)


def main():
    torch.set_num_threads(os.cpu_count() or 1)
    bind = load_binding()
    only = set(sys.argv[1:])   # optional: regenerate just the named cases
    for name, c in CASES.items():
        if only and name not in only:
            continue
        base = synth.make_inputs(c["T"], c["E_local"], seed=c["seed"], local_expert_offset=c["offset"],
                                 skew=c["skew"], only_experts=[], heavy_tail=c.get("heavy", False))
        idx, w = bind._ds_routing_impl(base["routing_logits"], base["routing_bias"], base["routed_scaling_factor"])
        sidx, sw = sorted_routing(idx, w)
        rec = dict(topk_idx=sidx.numpy().astype(np.int16), topk_w=sw.numpy().astype(np.float32),
                   meta=np.array([c["T"], c["E_local"], c["offset"], c["seed"], int(c["skew"]), int(c["full"]),
                                  int(c.get("heavy", False))]))
        if c["full"]:
            local = idx - c["offset"]
            hit = sorted(set(local[(local >= 0) & (local < c["E_local"])].tolist()))
            inp = synth.make_inputs(c["T"], c["E_local"], seed=c["seed"], local_expert_offset=c["offset"],
                                    skew=c["skew"], only_experts=hit, heavy_tail=c.get("heavy", False))
            bind.E_LOCAL = c["E_local"]
            bind._buf_cache.clear()
            out = torch.zeros((c["T"], 7168), dtype=torch.float32)
            bind.kernel(inp["routing_logits"], inp["routing_bias"], inp["hidden_states"], inp["hidden_states_scale"],
                        inp["gemm1_weights"], inp["gemm1_weights_scale"], inp["gemm2_weights"],
                        inp["gemm2_weights_scale"], c["offset"], inp["routed_scaling_factor"], out)
            rec["out_f32"] = out.numpy()
            rec["hit_experts"] = np.array(hit, dtype=np.int16)
        np.savez_compressed(HERE / f"{name}.npz", **rec)
        print(name, "hit" if c["full"] else "", rec.get("hit_experts", ""), flush=True)


if __name__ == "__main__":
    main()
