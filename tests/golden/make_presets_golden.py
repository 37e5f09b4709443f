"""Writes reference_presets.json: the resolved ModelArgs fields of every preset of the reference's
four family tables (read from the reference's source with `ast`; nothing is executed).  Presets
whose keyword arguments the reference's own ModelArgs would reject are skipped.

    python tests/golden/make_presets_golden.py --reference /path/to/ladder-residual-inference
"""
import argparse
import ast
import json
import os

FIELDS = {"block_size": 2048, "vocab_size": 32000, "n_layer": 32, "n_head": 32, "dim": 4096, "intermediate_size": None,
          "n_local_heads": -1, "rope_base": 10000, "norm_eps": 1e-5, "rope_scaling": None, "semi_compiled_model": False}
DESYNC_FIELDS = {"reduce_pattern": None, "force_disable_last_all_reduce": False}


def resolve(kw, desync):
    allowed = dict(FIELDS, **(DESYNC_FIELDS if desync else {}))
    if any(k not in allowed for k in kw):
        return None
    f = dict(allowed, **kw)
    if f["n_local_heads"] == -1:
        f["n_local_heads"] = f["n_head"]
    if f["intermediate_size"] is None:
        n = int(2 * (4 * f["dim"]) / 3)
        f["intermediate_size"] = n if n % 256 == 0 else n + 256 - n % 256
    f["head_dim"] = f["dim"] // f["n_head"]
    if desync and f["reduce_pattern"] is None:
        f["reduce_pattern"] = [{"attention": False, "mlp": True} for _ in range(f["n_layer"])]
    return f


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    a = ap.parse_args()
    out = {}
    for family in ("ladder", "dense", "parallel", "desync"):
        tree = ast.parse(open(os.path.join(a.reference, "gpt_fast", f"gpt_{family}_TP.py")).read())
        table = {}
        for node in tree.body:
            if isinstance(node, ast.Assign) and getattr(node.targets[0], "id", "") == "transformer_configs":
                for k, v in zip(node.value.keys, node.value.values):
                    kw = eval(compile(ast.Expression(v), "<preset>", "eval"), {"dict": dict, "range": range})
                    r = resolve(kw, family == "desync")
                    if r is not None:
                        table[k.value] = r
        out[family] = table
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_presets.json")
    json.dump(out, open(path, "w"), indent=0, sort_keys=True)
    print(path, {k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
