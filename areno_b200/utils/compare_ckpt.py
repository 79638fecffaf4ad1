"""Compare two Hugging Face safetensors checkpoints tensor by tensor.

    python -m areno_b200.utils.compare_ckpt BASE OTHER [--pattern 'model.layers.0.*'] [--top-k 30] [--json]

Reports keys present on one side only, shape / dtype mismatches and, for tensors both sides share, the
relative L2 difference, the largest absolute difference and the mean absolute difference, sorted by relative
difference.  Used when bringing up a model adapter (a saved checkpoint must reload to the same tensors) and to
see which parameters a training run moved.  Same purpose as the reference's
``skills/areno-model-adaptation/scripts/compare_ckpt_diff.py``; reads through this package's lazy index so
only one tensor pair is in memory at a time.
"""

from __future__ import annotations

import argparse
import fnmatch
import json

import torch

from ..engine.checkpoint import SafetensorsIndex


def _filter(keys, patterns):
    keys = sorted(keys)
    if not patterns:
        return keys
    return [k for k in keys if any(fnmatch.fnmatch(k, p) for p in patterns)]


def compare(base: str, other: str, patterns=(), max_elements: int = 0) -> dict:
    a, b = SafetensorsIndex(base), SafetensorsIndex(other)
    ka, kb = set(_filter(a.keys(), patterns)), set(_filter(b.keys(), patterns))
    report = {"base": base, "other": other, "missing_in_other": sorted(ka - kb), "extra_in_other": sorted(kb - ka),
              "shape_mismatch": [], "dtype_mismatch": [], "tensors": []}
    for n, key in enumerate(sorted(ka & kb)):
        ta, tb = a.get(key), b.get(key)
        if tuple(ta.shape) != tuple(tb.shape):
            report["shape_mismatch"].append({"key": key, "base": list(ta.shape), "other": list(tb.shape)})
            continue
        if ta.dtype != tb.dtype:
            report["dtype_mismatch"].append({"key": key, "base": str(ta.dtype), "other": str(tb.dtype)})
        fa, fb = ta.flatten().float(), tb.flatten().float()
        if max_elements and fa.numel() > max_elements:
            idx = torch.linspace(0, fa.numel() - 1, max_elements).long()
            fa, fb = fa[idx], fb[idx]
        diff = (fa - fb).abs()
        denom = float(fa.norm())
        report["tensors"].append({
            "key": key, "numel": int(ta.numel()), "rel_l2": float((fa - fb).norm()) / denom if denom > 0 else float(diff.sum() > 0),
            "max_abs": float(diff.max()) if diff.numel() else 0.0, "mean_abs": float(diff.mean()) if diff.numel() else 0.0})
        if n % 64 == 63:
            a.drop()
            b.drop()
    a.drop()
    b.drop()
    report["tensors"].sort(key=lambda r: (r["rel_l2"], r["max_abs"]), reverse=True)
    report["identical"] = (not report["missing_in_other"] and not report["extra_in_other"] and not report["shape_mismatch"]
                           and all(r["max_abs"] == 0.0 for r in report["tensors"]))
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("base")
    ap.add_argument("other")
    ap.add_argument("--pattern", action="append", default=[], help="fnmatch pattern of keys to include (repeatable)")
    ap.add_argument("--top-k", type=int, default=30)
    ap.add_argument("--max-elements", type=int, default=0, help="sample at most this many elements per tensor (0: all)")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    rep = compare(args.base, args.other, tuple(args.pattern), args.max_elements)
    if args.json:
        print(json.dumps(rep))
        return 0 if rep["identical"] else 1
    print(f"base={rep['base']}\nother={rep['other']}")
    for name in ("missing_in_other", "extra_in_other"):
        print(f"{name}: {len(rep[name])}" + ("" if not rep[name] else "  e.g. " + ", ".join(rep[name][:5])))
    for m in rep["shape_mismatch"]:
        print(f"shape mismatch {m['key']}: {m['base']} vs {m['other']}")
    for m in rep["dtype_mismatch"]:
        print(f"dtype mismatch {m['key']}: {m['base']} vs {m['other']}")
    print(f"compared {len(rep['tensors'])} tensors; identical={rep['identical']}")
    for r in rep["tensors"][: args.top_k]:
        print(f"{r['rel_l2']:.3e}  max {r['max_abs']:.3e}  mean {r['mean_abs']:.3e}  {r['key']}")
    return 0 if rep["identical"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
