"""TEST INFRASTRUCTURE -- CPU restatement (numpy) of the reference's constant fusion and of its
constants-section writers.  Nothing in the product imports this file.

Constant fusion (src/vpux_compiler/src/dialect/VPUIP/passes/fuse_constants.cpp:82-176,
populateFusedConstantBuffer): the constants of one NCE task -- weight table, weights, weights sparsity
map, activation window, in that order, absent ones skipped -- are folded and their values appended to one
byte vector: quantised and ui8 values byte by byte, f16 and si32 values as their little-endian bytes
(ConstantFusing::convertToU8), i1 content as its packed bytes.  The fused constant is typed f16
[1,1,1,total/2] when f16-typed constants hold more than half of the bytes, else ui8 [1,1,1,total].
Each original constant becomes a SubView of `size` elements at its running offset
(replaceConstantsWithFusedConstant :178-214).

Sections: the graph-schema writer gives every constant a zero-filled buffer of its size rounded up to 8 bytes
(serializeBinaryData, src/vpux_compiler/src/dialect/VPUIP/graph-schema/export.cpp:465-479); the ELF writer
appends the bytes with no padding (Const::DeclareOp::serialize, src/vpux_compiler/src/dialect/const/ops.cpp:97-108).
"""
import numpy as np


def fuse_constants(parts):
    """parts: list of (folded bytes as uint8 array, element kind) or None, in the order weight table, weights,
    weights sparsity map, activation window; kind in {"quant", "u8", "u8_from_f16", "f16", "si32", "i1"}.
    Returns (fused bytes, "f16" | "ui8", number of elements, [(offset, size) in elements of the fused type])."""
    total = sum(p[0].size for p in parts if p is not None)
    buf = []
    joint_f16 = 0
    for p in parts:
        if p is None:
            continue
        raw, kind = p
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        if kind in ("quant", "u8", "i1"):
            buf.append(raw)
        elif kind == "u8_from_f16":   # a compressed f16 constant seen as bytes
            buf.append(raw)
            joint_f16 += raw.size
        elif kind == "f16":
            buf.append(raw)           # two bytes per value, low byte first
            joint_f16 += raw.size
        elif kind == "si32":
            buf.append(raw)           # four bytes per value, low byte first
        else:
            raise ValueError(f"Unsupported data type for constant: {kind}")
    fused = np.concatenate(buf) if buf else np.zeros(0, np.uint8)
    assert fused.size == total
    if joint_f16 * 2 > total:
        elem, n, es = "f16", total // 2, 2
    else:
        elem, n, es = "ui8", total, 1
    views, off = [], 0
    for p in parts:
        if p is None:
            views.append(None)
            continue
        size = p[0].size // es
        views.append((off, size))
        off += size
    return fused, elem, n, views


def graph_schema_section(constants):
    """constants: list of uint8 arrays (the copyTo bytes).  Returns (section bytes, [offset of each])."""
    out, offs, at = [], [], 0
    for c in constants:
        padded = np.zeros((c.size + 7) // 8 * 8, np.uint8)
        padded[:c.size] = c
        out.append(padded)
        offs.append(at)
        at += padded.size
    return (np.concatenate(out) if out else np.zeros(0, np.uint8)), offs


def elf_section(constants):
    offs, at = [], 0
    for c in constants:
        offs.append(at)
        at += c.size
    return (np.concatenate(constants) if constants else np.zeros(0, np.uint8)), offs
