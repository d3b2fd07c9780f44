"""Extracts the constant-fusion known-answer vectors the reference pins in its lit test
tests/lit/NPU/dialect/VPUIP/passes/fuse_constants.mlir (read as text; nothing is executed) into
tests/golden/fuse_constants_vectors.json.  Run once where the reference tree is present:

    python tests/golden/make_fusion_vectors.py /path/to/reference
"""
import json
import os
import re
import sys


def main(ref):
    path = os.path.join(ref, "tests/lit/NPU/dialect/VPUIP/passes/fuse_constants.mlir")
    text = open(path).read()
    cases = []
    for block in text.split("// -----"):
        m = re.search(r"CHECK-LABEL: @(\w+)", block)
        if not m:
            continue
        name = m.group(1)
        fused = re.search(r"\[\[FUSED_CONSTANT:%\.\+\]\] = const\.Declare memref<1x1x1x(\d+)x(ui8|f16)>(?: = dense<\"0x([0-9A-Fa-f]+)\")?", block)
        if not fused:
            continue
        case = {"name": name, "fused_elems": int(fused.group(1)), "fused_elem_type": fused.group(2), "fused_hex": fused.group(3),
                "line": text[:text.index("@" + name)].count("\n") + 1, "constants": {}}
        for var, key in (("weight_table", "weight_table"), ("weights", "weights"), ("weights_sm", "weights_sm"),
                         ("act_wind", "activation_window")):
            d = re.search(r"%" + var + r" = const\.Declare [^=]+= dense<([^>]*)> : tensor<([0-9x]+)x(\w+)>(?:, \[([^\]]*)\])?", block)
            if not d:
                d2 = re.search(r"%" + var + r" = const\.Declare memref<([0-9x]+)x([!\w]+)(?:, #NHWC)?> = dense<([^>]*)>", block)
                if not d2:
                    continue
                shape, elem, value, chain = d2.group(1), d2.group(2), d2.group(3), None
                order = "NHWC" if "#NHWC>" in block[d2.start():d2.start() + 80] else "NCHW"
            else:
                value, shape, elem, chain = d.group(1), d.group(2), d.group(3), d.group(4)
                order = "NCHW"
            entry = {"shape": [int(s) for s in shape.split("x")], "elem": elem, "order": order,
                     "transforms": [t.strip() for t in chain.split(",")] if chain else []}
            value = value.strip()
            if value.startswith('"0x'):
                entry["hex"] = value[3:-1]
            elif value.startswith("["):
                entry["values"] = [int(v) for v in re.findall(r"-?\d+", value)]
            else:
                entry["splat"] = float(value)
            case["constants"][key] = entry
        q = re.search(r"!qElemType = !quant\.uniform<(\w+)<(-?\d+):(-?\d+)>:(\w+), ([0-9.eE+-]+)>", block)
        if q:
            case["qElemType"] = {"storage": q.group(1), "qmin": int(q.group(2)), "qmax": int(q.group(3)),
                                 "expressed": q.group(4), "scale": float(q.group(5))}
        cases.append(case)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fuse_constants_vectors.json")
    with open(out, "w") as f:
        json.dump({"source": "tests/lit/NPU/dialect/VPUIP/passes/fuse_constants.mlir", "cases": cases}, f, indent=1)
    print(f"{len(cases)} cases -> {out}")
    for c in cases:
        print(c["name"], c["line"], c["fused_elems"], c["fused_elem_type"], sorted(c["constants"]), "hex" if c["fused_hex"] else "")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
