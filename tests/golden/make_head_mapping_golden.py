"""Generate tests/golden/head_mapping.npz by executing the reference's own layer-selection code
(runners/stats_runner.py: _accumulate_similarity / _similarity_layer, _pick_k_layers, _get_pivot_score,
_find_head_mappings) on seeded synthetic attention statistics.

    python tests/golden/make_head_mapping_golden.py --reference /path/to/kascade

The runner module imports `accelerate` and `matplotlib` at module level for its other duties; neither is
needed by the four functions used here, so missing ones are replaced by empty stand-in modules for the
import.  The functions are called unbound on a small attribute holder instead of a full runner.
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests.test_head_mapping_cpu import NUM_LAYERS, HEADS, PROMPTS, synthetic_stats, synthetic_importance  # noqa: E402


def load_stats_runner(path):
    for name in ("accelerate", "accelerate.utils", "matplotlib", "matplotlib.pyplot"):
        try:
            importlib.import_module(name)
        except Exception:
            stub = types.ModuleType(name)
            stub.Accelerator = object
            stub.reduce = stub.gather_object = lambda *a, **k: None
            sys.modules[name] = stub
    src = os.path.join(path, "src")
    pkg = types.ModuleType("kascade_runners")
    pkg.__path__ = [os.path.join(src, "runners")]
    sys.modules["kascade_runners"] = pkg
    base = types.ModuleType("kascade_runners.base")                 # the runner base class is not exercised
    base.BaseGenerationRunner = object
    base.GenerationStep = object
    sys.modules["kascade_runners.base"] = base
    spec = importlib.util.spec_from_file_location("kascade_runners.stats_runner",
                                                  os.path.join(src, "runners", "stats_runner.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["kascade_runners.stats_runner"] = mod
    spec.loader.exec_module(mod)
    return mod.StatsRunner


class Holder:
    pass


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    SR = load_stats_runner(args.reference)
    out = {}
    for reduce, run_type in (("amin", "select_layers"), ("mean", "plot_similarity")):
        h = Holder()
        h.config = Holder()
        h.config.run_type = run_type
        h._post_processing_type = run_type
        h._num_layers = NUM_LAYERS
        h._sim_mat = torch.zeros(NUM_LAYERS, NUM_LAYERS, HEADS, HEADS)
        h._similarity_layer = lambda a, b, h=h: SR._similarity_layer(h, a, b)
        for p in range(PROMPTS):
            idx, w, last = synthetic_stats(p)
            h._top_k_per_layer, h._causal_attn_weights, h._last_tile_attn = idx, w, last
            SR._accumulate_similarity(h)
        sim_avg = h._sim_mat / PROMPTS
        out[f"sim_avg_{reduce}"] = sim_avg.numpy()
    sim_avg = torch.from_numpy(out["sim_avg_amin"])
    imp = synthetic_importance()
    layer_sim = (sim_avg.amax(dim=-1).mean(dim=-1) * imp.unsqueeze(0)).cpu().numpy()      # stats_runner.py:186-187
    out["layer_sim"] = layer_sim
    h = Holder()
    h._num_layers = NUM_LAYERS
    for K in (3, 4, 5, 6, 7, 8):
        pivots = SR._pick_k_layers(h, layer_sim, K)
        out[f"pivots_{K}"] = np.array(pivots, dtype=np.int32)
        out[f"score_{K}"] = np.array(SR._get_pivot_score(h, layer_sim, pivots + [NUM_LAYERS]), dtype=np.float64)
        import contextlib
        import io
        with contextlib.redirect_stdout(io.StringIO()):
            out[f"mapping_{K}"] = np.array(SR._find_head_mappings(h, sim_avg, pivots + [NUM_LAYERS]), dtype=np.int32)
    path = os.path.join(HERE, "head_mapping.npz")
    np.savez_compressed(path, **out)
    print(path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
