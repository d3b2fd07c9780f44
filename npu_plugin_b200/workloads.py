"""The five benchmark workloads as lists of constant declarations, with their seeded synthetic inputs.

Shapes, chains and value distributions follow the benchmark configurations: a conv weight folded to
swizzled int8, an int4 weight-only linear layer with its dequantise leg, a 50 % sparse 1x1 conv weight
(sparsity map + sparsify), a ResNet-50-shaped int8 weight set under the block codec and a 7B
Llama-shaped decoder, as plain descriptor lists (no data, no backend).  The reference's own chain-building
call sites are restated in npu_plugin_b200.chains.
No dataset is involved: every input comes from the counter-based generator behind b200c_synth_fill,
keyed by (SEED, stream id of the constant).
"""
from . import _cabi as A
from .blob import ConstantDecl
from .const import DimsOrder, NDType, Transform, UniformQuantizedPerAxisType, UniformQuantizedType

SEED = 5


def _decl(name, base_type, chain, nbytes, compress, synth, stream):
    d = ConstantDecl(name, base_type, chain, nbytes, compress=compress)
    d.synth = synth      # (dtype, distribution, p0, p1) of b200c_synth_fill
    d.stream = stream    # generator stream: constants sharing a stream hold the same values
    return d


def llama7b_decls(layers=32, hidden=4096, ffn=11008, vocab=32000):
    """7 linear weights per layer + lm_head (symmetric int8 per channel -> Reorder -> Swizzle(5) -> codec),
    the embedding and 2 * layers + 1 RMSNorm gains (f16, empty chain, not compressed)."""
    decls = []

    def linear(name, o, i):
        q = UniformQuantizedPerAxisType(A.SI8, A.F16, [1.0] * o, [0] * o, 0, -127, 127)
        chain = [Transform(A.X_QUANTIZE_SYNTH, i0=A.QSYNTH_SYM_I8), Transform(A.X_CONVERT_ELEM_TYPE, elem=A.SI8),
                 Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.NHWC),
                 Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]
        decls.append(_decl(name, NDType((o, i, 1, 1), A.F16), chain, o * i * 2, True, (A.F16, 0, 0.02, 0.0), len(decls)))

    for l in range(layers):
        for n in ("q", "k", "v", "o"):
            linear(f"l{l}.{n}", hidden, hidden)
        linear(f"l{l}.gate", ffn, hidden)
        linear(f"l{l}.up", ffn, hidden)
        linear(f"l{l}.down", hidden, ffn)
    linear("lm_head", vocab, hidden)
    decls.append(_decl("embedding", NDType((vocab, hidden), A.F16), [], vocab * hidden * 2, False, (A.F16, 0, 1.0, 0.0),
                       len(decls)))
    for l in range(2 * layers + 1):
        decls.append(_decl(f"norm{l}", NDType((hidden,), A.F16), [], hidden * 2, False, (A.F16, 0, 1.0, 0.0), len(decls)))
    return decls


def conv_weight_decls(instances):
    """f32 [256,256,3,3] -> symmetric int8 per channel -> OIYX->OYXI -> pad I to a multiple of 16 -> Swizzle(5)."""
    decls = []
    for k in range(instances):
        q = UniformQuantizedPerAxisType(A.SI8, A.F32, [1.0] * 256, [0] * 256, 0, -127, 127)
        chain = [Transform(A.X_QUANTIZE_SYNTH, i0=A.QSYNTH_SYM_I8), Transform(A.X_CONVERT_ELEM_TYPE, elem=A.SI8),
                 Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.OYXI),
                 Transform(A.X_PAD_WITH_ZERO, a=(0, 0, 0, 0), b=(0, 0, 0, 0)), Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]
        decls.append(_decl(f"conv{k}", NDType((256, 256, 3, 3), A.F32), chain, 256 * 256 * 9 * 4, False,
                           (A.F32, 0, 0.05, 0.0), k))
    return decls


def int4_linear_decls(instances, O=11008, I=4096):
    """f16 [O,I] -> asymmetric u4 per channel -> NHWC -> BitPack; and the dequantise leg u8 [O,I] ->
    per-axis QuantCast -> Dequantize -> f16."""
    decls = []
    for k in range(instances):
        q = UniformQuantizedPerAxisType(A.UI8, A.F16, [1.0] * O, [0] * O, 0, 0, 15)
        chain = [Transform(A.X_QUANTIZE_SYNTH, i0=A.QSYNTH_ASYM_U4), Transform(A.X_CONVERT_ELEM_TYPE, elem=A.UI8),
                 Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.NHWC), Transform(A.X_BIT_PACK, i0=4)]
        decls.append(_decl(f"pack{k}", NDType((O, I, 1, 1), A.F16), chain, O * I * 2, False, (A.F16, 0, 0.02, 0.0), 2 * k))
        qd = UniformQuantizedPerAxisType(A.UI8, A.F16, [0.001 + 1e-6 * (j % 97) for j in range(O)], [j % 16 for j in range(O)],
                                         0, 0, 15)
        chain = [Transform(A.X_QUANT_CAST, elem=qd), Transform(A.X_REORDER, a=DimsOrder.NHWC), Transform(A.X_DEQUANTIZE)]
        decls.append(_decl(f"dequant{k}", NDType((O, I, 1, 1), A.UI8), chain, O * I, False, (A.SI8, 1, 0.0, 0.0), 2 * k + 1))
    return decls


def sparse_conv_decls(instances):
    """int8 [1024,1024,1,1] with 50 % zeros -> GetSparsityMap -> Swizzle(5), and -> Sparsify -> Swizzle(5);
    both chains of an instance read the same weights."""
    decls = []
    for k in range(instances):
        for name, chain in (("map", [Transform(A.X_GET_SPARSITY_MAP), Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)]),
                            ("vals", [Transform(A.X_SPARSIFY, i0=0), Transform(A.X_SWIZZLE_CONSTANT, i0=5, i1=3)])):
            decls.append(_decl(f"{name}{k}", NDType((1024, 1024, 1, 1), A.SI8), chain, 1024 * 1024, False,
                               (A.SI8, 1, 0.5, 0.0), k))
    return decls


def resnet50_shapes():
    shapes = [(64, 3, 7, 7)]
    inplanes = 64
    for width, blocks in ((64, 3), (128, 4), (256, 6), (512, 3)):
        for b in range(blocks):
            shapes += [(width, inplanes, 1, 1), (width, width, 3, 3), (width * 4, width, 1, 1)]
            if b == 0:
                shapes.append((width * 4, inplanes, 1, 1))
            inplanes = width * 4
    shapes.append((1000, 2048, 1, 1))
    return shapes


def resnet_decls(instances):
    """53 conv + fc int8 weights -> QuantCast -> OIYX->OYXI (-> pad I to a multiple of 16) -> block codec."""
    decls = []
    for k in range(instances):
        for j, (o, i, y, x) in enumerate(resnet50_shapes()):
            q = UniformQuantizedType(A.SI8, A.F16, 0.01, 0, -127, 127)
            chain = [Transform(A.X_QUANT_CAST, elem=q), Transform(A.X_REORDER, a=DimsOrder.OYXI)]
            if i % 16 and i < 16:
                chain.append(Transform(A.X_PAD_WITH_ZERO, a=(0, 0, 0, 0), b=(0, 16 - i % 16, 0, 0)))
            decls.append(_decl(f"r{k}.{j}", NDType((o, i, y, x), A.SI8), chain, o * i * y * x, True, (A.SI8, 2, 12.0, 0.1),
                               len(decls)))
    return decls


# name -> (builder, default instances per step, description, arithmetic type, dominant kernel of the workload)
WORKLOADS = {
    "cfg1": (conv_weight_decls, 512, "conv weight f32 [256,256,3,3] -> sym int8 -> OYXI -> pad -> Swizzle(5)", "f32->i8",
             "rowQuantSmemBatchKernel"),
    "cfg2": (int4_linear_decls, 8, "f16 [11008,4096] -> asym u4 -> BitPack; and u8 -> per-axis Dequantize -> f16", "f16->u4",
             "rowQuantRegBatchKernel"),
    "cfg3": (sparse_conv_decls, 512, "int8 [1024,1024,1,1] 50% sparse -> sparsity map + sparsify, both Swizzle(5)", "i8",
             "sparseScatterBatchKernel"),
    "cfg4": (resnet_decls, 32, "ResNet-50-shaped int8 set (54 tensors) -> QuantCast -> OYXI (-> pad) -> block codec", "i8",
             "codecEmitKernel"),
}


# chunks a single rank cuts the workload into: with several, the device compresses chunk k while the host plans
# the fold of chunk k + 1 (worth it where the constants are small and every one of them is compressed)
PIPELINE_CHUNKS = {}


def has_quantizer(d):
    return any(t.kind == A.X_QUANTIZE_SYNTH for t in d.transforms)


def shared_inputs(decls):
    """Constants that hold the same values (same generator stream, type and size: the sparsity map and the
    sparsified values of one weight) share one base content, as the two DeclareOps of a sparse weight share one
    dense resource in the compiler.  Returns (owner index per constant, indices that own a buffer)."""
    first, owner = {}, []
    for i, d in enumerate(decls):
        key = (d.stream, d.nbytes, tuple(d.synth), d.base_type.dtype)
        owner.append(first.setdefault(key, i))
    return owner, sorted(set(owner))


def fill_device(backend, d, dev_ptr):
    """Writes the constant's synthetic values into device memory with the library's generator."""
    dt, dist, p0, p1 = d.synth
    backend.synth_fill(dev_ptr, d.nbytes * 8 // A.dtype_bits(dt), dt, dist, p0, p1, SEED, d.stream)


def algorithmic_bytes(decls, folded_sizes, stream_sizes, slot_sizes=None):
    """Read-once + write-once bytes of one step.  Fold: input + folded output (the bytes really written into the
    blob slot: folded_sizes) + the quantiser's scale tables.  Codec: every constant offered to it is read once
    (its whole slot: slot_sizes, default folded_sizes); only a stream that is smaller than its constant is written
    (stream_sizes[i] is its length, else None)."""
    fold = sum(d.nbytes for d in decls) + sum(folded_sizes)
    fold += sum(4 * d.base_type.shape[0] for d in decls if has_quantizer(d))
    codec = 0
    for d, fs, ss in zip(decls, slot_sizes if slot_sizes is not None else folded_sizes, stream_sizes):
        if d.compress and fs >= 4096:
            codec += fs + (ss or 0)
    return fold, codec
