"""Generate the golden vectors under tests/golden/ by executing the reference's own PyTorch
``KascadeStrategy`` (strategies/KascadeStrategy.py) on seeded inputs.

Runs only where a checkout of the reference is available:

    python tests/golden/make_golden.py --reference /path/to/kascade

The reference is imported unmodified through a package alias (its pyproject maps the package name
``kascade`` onto ``src/``).  Inputs are drawn in fp32, rounded to fp16 and converted back, so the
fp32 reference and fp16 CUDA kernels see bit-identical values.  Only the seeds, a checksum of the
inputs, the index rows and (sub-sampled) outputs are stored, so the files stay small.
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from tests.cases import CASES, make_inputs, decode_inputs, input_checksum  # noqa: E402


def load_reference(path):
    src = os.path.join(path, "src")
    spec = importlib.util.spec_from_file_location(
        "kascade", os.path.join(src, "__init__.py"), submodule_search_locations=[src])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["kascade"] = mod
    spec.loader.exec_module(mod)
    return importlib.import_module("kascade.strategies.KascadeStrategy").KascadeStrategy


class _Module:
    training = False

    def __init__(self, layer_idx, groups):
        self.layer_idx = layer_idx
        self.num_key_value_groups = groups


def run_case(KS, case, workdir):
    c = case
    os.makedirs(os.path.join(workdir, "results", "head_mappings"), exist_ok=True)
    mapping = np.asarray(c.head_mapping(), dtype=np.int32)
    name = f"golden_{c.name}"
    np.save(os.path.join(workdir, "results", "head_mappings",
                         f"{name}_layers_{'_'.join(map(str, c.anchors))}.npy"), mapping)
    cwd = os.getcwd()
    os.chdir(workdir)
    try:
        strat = KS(recompute_layers=list(c.anchors), model_name=f"x/{name}", k=c.pct,
                   tile_size=c.tile, rolling_prefill=c.rolling, block_size=c.block_size)
    finally:
        os.chdir(cwd)
    out = {"checksum": np.float64(0.0)}
    hg = c.H // c.G
    scaling = c.D ** -0.5
    fmin = torch.finfo(torch.float32).min
    mask = torch.full((c.L, c.L), fmin).triu_(1)[None, None].expand(c.B, 1, c.L, c.L).contiguous()
    qsel = torch.tensor(c.sampled_queries())
    cks = 0.0
    for layer in range(c.layers):
        q, k, v = make_inputs(c, layer)
        cks += input_checksum(q, k, v)
        o, _ = strat.attention_forward(_Module(layer, hg), q, k, v, mask, scaling)
        out[f"prefill_out_{layer}"] = o[:, qsel].to(torch.float16).numpy()
        if layer == 0 or layer in c.anchors:
            out[f"prefill_idx_{layer}"] = strat._topk_to_reuse[:, :, ::c.tile].numpy().astype(np.int32)
    # one decode step at position L (strategies/KascadeStrategy.py: Lq == 1 path)
    dmask = torch.zeros(c.B, 1, 1, c.L + 1)
    for layer in range(c.layers):
        q, k, v = decode_inputs(c, layer)
        cks += input_checksum(q, k, v)
        o, _ = strat.attention_forward(_Module(layer, hg), q, k, v, dmask, scaling)
        out[f"decode_out_{layer}"] = o.to(torch.float32).numpy()
        if layer == 0 or layer in c.anchors:
            out[f"decode_idx_{layer}"] = strat._topk_to_reuse[:, :, 0].numpy().astype(np.int32)
    out["checksum"] = np.float64(cks)
    out["sampled_queries"] = qsel.numpy().astype(np.int32)
    out["head_mapping"] = mapping
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of microsoft/kascade (read only)")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    KS = load_reference(args.reference)
    torch.set_grad_enabled(False)
    for case in CASES:
        if args.only and case.name != args.only:
            continue
        with tempfile.TemporaryDirectory() as wd:
            res = run_case(KS, case, wd)
        path = os.path.join(HERE, f"{case.name}.npz")
        np.savez_compressed(path, **res)
        print(case.name, "->", path, f"{os.path.getsize(path) / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
