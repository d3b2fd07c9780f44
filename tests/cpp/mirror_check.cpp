// Exercises the C++ host layer (include/b200const.hpp) the way the reference's unit tests exercise
// vpux::Const::ContentAttr (tests/unit/vpux_compiler/dialect/const/content_tests.cpp): build an
// attribute, add transformations, fold, compare with a plain-loop expectation written here.
// Exit code 0 = all checks passed; each failure prints one line.
#include "b200const.hpp"

#include <cmath>
#include <cstdio>
#include <numeric>
#include <random>

using namespace b200::Const;

static int failures = 0;
#define EXPECT(cond, what)                                  \
    do {                                                    \
        if (!(cond)) {                                      \
            std::printf("FAILED: %s (%s)\n", what, #cond);  \
            ++failures;                                     \
        }                                                   \
    } while (0)

int main() {
    // ---- host-only part: insertion order and type inference (content_tests.cpp:1342-1393) ----
    {
        std::vector<float> vals(2 * 16 * 3 * 3);
        std::iota(vals.begin(), vals.end(), 0.0f);
        auto a = ContentAttr::get(vals, NDType({2, 16, 3, 3}, B200C_F32));
        auto b = a.swizzleConstant(5, 3).getSparsityMap().rescale(2.0);  // added out of order on purpose
        EXPECT(b.getNumTransformations() == 3, "three transformations");
        EXPECT(b.getTransformationKind(0) == B200C_X_RESCALE, "NONE first");
        EXPECT(b.getTransformationKind(1) == B200C_X_GET_SPARSITY_MAP, "PREFERRED_LAST second");
        EXPECT(b.getTransformationKind(2) == B200C_X_SWIZZLE_CONSTANT, "LAST last");
        bool threw = false;
        try {
            b.bitPack(4);
        } catch (const Error& e) {
            threw = e.code() == B200C_ERR_THROW;
        }
        EXPECT(threw, "a second LAST transformation throws");
        const NDType t = a.reorder(DimsOrder::NHWC()).padWithZero({0, 0, 0, 0}, {0, 16, 0, 0}).getType();
        EXPECT((t.shape == std::vector<int64_t>{2, 32, 3, 3}) && t.order == DimsOrder::NHWC(), "inferred type of reorder + pad");
    }
    // ---- Const::DeclareOp verifier (ops.cpp:164-193), host only ----
    {
        std::vector<float> vals(12);
        std::iota(vals.begin(), vals.end(), 0.0f);
        auto a = ContentAttr::get(vals, NDType({3, 4}, B200C_F32));
        auto throws = [&](const NDType& t, const ContentAttr& attr, bool swizzled = false) {
            try {
                DeclareOp op(t, attr, swizzled);
            } catch (const Error& e) {
                return e.code() == B200C_ERR_THROW;
            }
            return false;
        };
        EXPECT(throws(NDType({4, 3}, B200C_F32), a), "DeclareOp: shape mismatch");
        EXPECT(throws(NDType({3, 4}, B200C_F16), a), "DeclareOp: element type mismatch");
        EXPECT(throws(NDType({3, 4}, B200C_F32, DimsOrder::fromPermutation({1, 0})), a), "DeclareOp: order mismatch");
        EXPECT(!throws(NDType({3, 4}, B200C_F32), a), "DeclareOp: matching type");
        std::vector<uint8_t> bytes(100);
        auto sw = ContentAttr::get(bytes, NDType({1, 100, 1, 1}, B200C_UI8)).swizzleConstant(5, 3);
        EXPECT(throws(NDType({1, 100, 1, 1}, B200C_UI8), sw), "DeclareOp: flattened swizzled content needs the swizzled flag");
        EXPECT(!throws(NDType({1, 100, 1, 1}, B200C_UI8), sw, true), "DeclareOp: swizzled result type skips the shape check");
        EXPECT(DeclareOp(NDType({1, 100, 1, 1}, B200C_UI8), sw, true).getBinarySize() == 512, "getBinarySize of a swizzled constant");
    }
    // ---- ContentAttr::verify on a dense resource (content.cpp:61-99; lit content.mlir:70-136), host only ----
    {
        auto refused = [&](const std::vector<uint32_t>& words, const NDType& t, const char* size) {
            try {
                ContentAttr::get(words, t);
            } catch (const Error& e) {
                return e.code() == B200C_ERR_THROW &&
                       std::string(e.what()).find(std::string("Size of dense resource buffer '") + size + "'") != std::string::npos;
            }
            return false;
        };
        const NDType t({1, 3, 1, 1}, B200C_F32);
        EXPECT(!ContentAttr::get(std::vector<uint32_t>{1, 2, 3}, t).isSplat(), "verify: a full dense resource");
        EXPECT(refused({2, 3}, t, "8"), "verify: 8 bytes for three f32");
        EXPECT(refused({1, 2, 3, 4}, t, "16"), "verify: 16 bytes for three f32");
        EXPECT(ContentAttr::get(std::vector<uint32_t>{1}, NDType({2, 3, 1, 1}, B200C_F32)).isSplat(), "verify: one element is a splat");
        EXPECT(!ContentAttr::get(std::vector<uint32_t>{1}, NDType({1}, B200C_F32)).isSplat(), "verify: a one-element type is no splat");
        const NDType bits({4, 8}, B200C_I1);
        EXPECT(ContentAttr::get(std::vector<uint8_t>{0xFF}, bits).isSplat(), "verify: 0xFF is a one-bit splat");
        bool threw = false;
        try {
            ContentAttr::get(std::vector<uint8_t>{0x0F}, bits);
        } catch (const Error&) {
            threw = true;
        }
        EXPECT(threw, "verify: a lone byte of mixed bits is refused");
    }
    // ---- stripTransformationsFrom / getLastTransformationsFrom (content_tests.cpp:1739-1796), host only ----
    {
        std::vector<float> vals(10);
        std::iota(vals.begin(), vals.end(), 0.0f);
        auto a = ContentAttr::get(vals, NDType({10}, B200C_F32)).add(1.0).reshape({2, 5}).subview({0, 0}, {1, 5});
        EXPECT(a.getNumTransformations() == 3, "Add, Reshape, SubView");
        auto head = a.stripTransformationsFrom(1);
        EXPECT(head.getNumTransformations() == 1 && head.getTransformationKind(0) == B200C_X_ADD, "head of the list is Add");
        EXPECT((a.getLastTransformationsFrom(1) == std::vector<int>{B200C_X_RESHAPE, B200C_X_SUBVIEW}), "tail is Reshape, SubView");
        // two equal Reshapes are one object in the reference: either of them cuts at the second
        auto d = ContentAttr::get(vals, NDType({10}, B200C_F32)).add(1.0).reshape({2, 5}).reshape({2, 5}).subview({0, 0}, {1, 5});
        EXPECT(d.getNumTransformations() == 4 && d.sameTransformation(1, 2), "duplicated Reshape");
        for (size_t which : {size_t(1), size_t(2)}) {
            auto h = d.stripTransformationsFrom(which);
            EXPECT(h.getNumTransformations() == 2 && h.getTransformationKind(1) == B200C_X_RESHAPE, "head is Add, Reshape");
            EXPECT((d.getLastTransformationsFrom(which) == std::vector<int>{B200C_X_RESHAPE, B200C_X_SUBVIEW}), "tail is Reshape, SubView");
        }
    }
    // ---- chain builders (const_utils.cpp:101-119,246-283; convert_weights_to_u8.cpp:85-101; hwtest_utils.cpp:184-197;
    //      swizzling.cpp:469-500; flatten_sparse_weights_types.cpp:41-73): lists and inferred types, host only ----
    {
        auto kinds = [](const ContentAttr& a) {
            std::vector<int> k;
            for (size_t i = 0; i < a.getNumTransformations(); ++i) k.push_back(a.getTransformationKind(i));
            return k;
        };
        std::vector<int8_t> w(8 * 3 * 3 * 3);
        for (size_t i = 0; i < w.size(); ++i) w[i] = static_cast<int8_t>(i % 101) - 50;
        const auto base = ContentAttr::get(w, NDType({8, 3, 3, 3}, B200C_SI8));
        const auto a = chains::alignConvolutionWeights(base, 16);
        EXPECT((kinds(a) == std::vector<int>{B200C_X_RESHAPE, B200C_X_PAD_WITH_ZERO}), "aligned weights: Reshape, PadWithZero");
        EXPECT((a.getType().shape == std::vector<int64_t>{8, 1, 1, 32}), "aligned weights: [8,1,1,32]");
        const auto c = chains::alignConvolutionWeights(base, 16, true);
        EXPECT((kinds(c) == std::vector<int>{B200C_X_REORDER, B200C_X_RESHAPE, B200C_X_PAD_WITH_ZERO, B200C_X_REORDER}),
               "C-major aligned weights: Reorder, Reshape, PadWithZero, Reorder");
        EXPECT((c.getType().shape == std::vector<int64_t>{8, 1, 1, 32}) && c.getType().order == DimsOrder::NHWC(), "C-major aligned weights: NHWC");
        std::vector<int8_t> w16(4 * 16);
        EXPECT(chains::alignConvolutionWeights(ContentAttr::get(w16, NDType({4, 16, 1, 1}, B200C_SI8))).getNumTransformations() == 0,
               "aligned already: untouched");
        std::vector<uint16_t> dw(6 * 9);
        const auto d = chains::alignDepthwiseWeights(ContentAttr::get(dw, NDType({6, 1, 3, 3}, B200C_F16)), {6, 9, 1, 1}, 7);
        EXPECT((d.getType().shape == std::vector<int64_t>{6, 16, 1, 1}) && d.getType().order == DimsOrder::NHWC(), "depthwise weights: [6,16,1,1] NHWC");
        // i8 -> u8
        std::vector<int8_t> q8(4 * 8);
        const QuantParams qs = QuantParams::perTensor(B200C_F16, 0.02, -3, -128, 127), qu = QuantParams::perTensor(B200C_F16, 0.02, 125, 0, 255);
        const auto u = chains::weightsToU8(ContentAttr::get(q8, NDType({4, 8, 1, 1}, B200C_SI8)).quantCast(qs, B200C_SI8), qu);
        EXPECT((kinds(u) == std::vector<int>{B200C_X_QUANT_CAST, B200C_X_QUANT_CAST, B200C_X_CONVERT_ELEM_TYPE, B200C_X_ADD,
                                             B200C_X_CONVERT_ELEM_TYPE, B200C_X_QUANT_CAST}),
               "weights to u8: QuantCast, ConvertElemType, Add, ConvertElemType, QuantCast behind the constant's own QuantCast");
        const NDType ut = u.getType();
        EXPECT(ut.dtype == B200C_UI8 && ut.quant.kind == B200C_Q_PER_TENSOR && ut.quant.zps == qu.zps && ut.quant.scales == qu.scales,
               "weights to u8: the new quantised type");
        bool threw = false;
        try {
            chains::weightsToU8(ContentAttr::get(q8, NDType({4, 8, 1, 1}, B200C_SI8)), qu);
        } catch (const Error&) {
            threw = true;
        }
        EXPECT(threw, "weights to u8 needs a quantised constant");
        // hardware-test weights
        std::vector<uint8_t> hw(2 * 4 * 1 * 2);
        const QuantParams q4 = QuantParams::perTensor(B200C_F16, 0.5, 0, 0, 15);
        const auto h = chains::hwtestDefaultWeights(ContentAttr::get(hw, NDType({2, 4, 1, 2}, B200C_UI8)), &q4, B200C_UI4);
        EXPECT((kinds(h) == std::vector<int>{B200C_X_REORDER, B200C_X_QUANT_CAST, B200C_X_BIT_PACK}), "hw-test weights: Reorder, QuantCast, BitPack");
        EXPECT((kinds(chains::hwtestDefaultWeights(ContentAttr::get(hw, NDType({2, 4, 1, 2}, B200C_UI8)))) == std::vector<int>{B200C_X_REORDER}),
               "hw-test weights without a quantised type: Reorder");
        // swizzle once
        std::vector<uint8_t> sw(1024);
        const auto s1 = chains::attachSwizzle(ContentAttr::get(sw, NDType({4, 256, 1, 1}, B200C_UI8)));
        EXPECT((kinds(s1) == std::vector<int>{B200C_X_SWIZZLE_CONSTANT}) && kinds(chains::attachSwizzle(s1)) == kinds(s1), "SwizzleConstant is attached once");
        // Sparsify<false> -> Sparsify<true, numElems>: the flat compressed type
        std::vector<int8_t> sp(16 * 32);
        const auto vals = ContentAttr::get(sp, NDType({16, 32, 1, 1}, B200C_SI8)).sparsify(false);
        std::vector<int64_t> counts(16);
        int64_t total = 0;
        for (int o = 0; o < 16; ++o) {
            counts[o] = o + 1;
            total += (counts[o] + 15) / 16 * 16;
        }
        EXPECT((chains::flattenSparseWeights(vals, counts).getType().shape == std::vector<int64_t>{total, 1, 1, 1}), "flattened sparse weights: [sum of 16-byte aligned runs,1,1,1]");
        EXPECT((vals.getType().shape == std::vector<int64_t>{16, 32, 1, 1}), "Sparsify<false> keeps the shape");
    }
    if (std::getenv("B200C_MIRROR_HOST_ONLY")) {
        std::printf("%s (host-only part)\n", failures ? "FAILED" : "OK");
        return failures ? 1 : 0;
    }

    Backend be(0);
    // ---- ConvertElemType + Reorder + PadWithZero + Add, f32 -> checked casts (content_tests.cpp style) ----
    {
        const std::vector<int64_t> shape{2, 3, 2, 2};
        std::vector<float> vals(24);
        std::iota(vals.begin(), vals.end(), 0.0f);
        auto c = ContentAttr::get(vals, NDType(shape, B200C_F32))
                         .add(1.0)
                         .reorder(DimsOrder::NHWC())
                         .padWithZero({0, 0, 0, 0}, {0, 1, 0, 0})
                         .convertElemType(B200C_SI8)
                         .fold(be);
        EXPECT((c.getType().shape == std::vector<int64_t>{2, 4, 2, 2}), "padded shape");
        const auto got = c.getValues<int8_t>();
        std::vector<int8_t> want;
        for (int n = 0; n < 2; ++n)
            for (int h = 0; h < 2; ++h)
                for (int w = 0; w < 2; ++w)
                    for (int ch = 0; ch < 4; ++ch)
                        want.push_back(ch < 3 ? static_cast<int8_t>(vals[((n * 3 + ch) * 2 + h) * 2 + w] + 1) : 0);
        EXPECT(got == want, "add + NHWC reorder + pad + convert");
    }
    // ---- per-axis Dequantize to f16-expressed type: float((q - zp) * double scale) ----
    {
        std::vector<uint8_t> q(4 * 8);
        for (size_t i = 0; i < q.size(); ++i) q[i] = static_cast<uint8_t>(i * 7);
        const std::vector<double> scales{0.5, 0.25, 2.0, 0.125};
        const std::vector<int64_t> zps{0, 3, 128, 255};
        auto c = ContentAttr::get(q, NDType({4, 8}, B200C_UI8))
                         .quantCast(QuantParams::perAxis(B200C_F32, scales, zps, 0, 0, 255), B200C_UI8)
                         .dequantize()
                         .fold(be);
        const auto got = c.getValues<float>();
        bool same = got.size() == q.size();
        for (size_t i = 0; same && i < q.size(); ++i)
            same = got[i] == static_cast<float>((static_cast<int64_t>(q[i]) - zps[i / 8]) * scales[i / 8]);
        EXPECT(same, "per-axis dequantize");
    }
    // ---- GetSparsityMap + Sparsify + countNonSparseElementsPerOC on a 50 % sparse int8 weight ----
    {
        std::mt19937 rng(7);
        std::vector<int8_t> w(8 * 32);
        for (auto& v : w) v = (rng() & 1) ? static_cast<int8_t>(static_cast<int>(rng() % 255) - 127) : 0;
        auto base = ContentAttr::get(w, NDType({8, 32, 1, 1}, B200C_SI8));
        const auto counts = base.countNonSparseElementsPerOC(be);
        const auto map = base.getSparsityMap().fold(be).getRawBytes();
        const auto vals = base.sparsify(false).fold(be).getRawBytes();
        bool ok = map.size() == 8 * 16 && counts.size() == 8;
        size_t at = 0;
        for (int oc = 0; ok && oc < 8; ++oc) {
            int64_t n = 0;
            for (int j = 0; j < 32; ++j) {
                const bool nz = w[oc * 32 + j] != 0;
                ok = ok && (((map[oc * 16 + j / 8] >> (j % 8)) & 1) == (nz ? 1 : 0));
                if (nz) {
                    ok = ok && at + n < vals.size() && static_cast<int8_t>(vals[at + n]) == w[oc * 32 + j];
                    ++n;
                }
            }
            ok = ok && counts[oc] == n;
            at += static_cast<size_t>((n + 15) / 16 * 16);
        }
        EXPECT(ok, "sparsity map (LSB first, rows padded to 128 bits), compacted values (16-byte channel starts), counts");
    }
    // ---- SwizzleConstant address rule (swizzle key 5) and the codec round trip ----
    {
        std::vector<uint8_t> x(4096);
        for (size_t i = 0; i < x.size(); ++i) x[i] = static_cast<uint8_t>((i / 16) & 0xFF);
        const auto sw = ContentAttr::get(x, NDType({4096, 1, 1, 1}, B200C_UI8)).swizzleConstant(5, 3).fold(be).getRawBytes();
        bool ok = sw.size() == 4096;
        for (size_t a = 0; ok && a < x.size(); a += 16) {
            const size_t block = (a >> 9) & 63, stagger = (block & 31) << 4;
            const size_t to = (a & ~size_t(511)) + ((a + stagger) & 511);
            ok = std::memcmp(&sw[to], &x[a], 16) == 0;
        }
        EXPECT(ok, "swizzle address rule");
        std::vector<uint8_t> stream;
        const bool smaller = compress(be, x, &stream);
        EXPECT(smaller && stream.size() < x.size(), "codec shrinks a ramp of 16-byte runs");
        EXPECT(decompress(be, stream, x.size()) == x, "codec round trip");
    }
    // ---- the constant-folding pass on a 4-bit constant (constant_folding.cpp:45-68; lit
    //      tests/lit/NPU/dialect/const/passes/constant_folding.mlir:212-222: bytes [16, 18], type 1x1x1x2xui8) ----
    {
        const DimsOrder YXOI = DimsOrder::fromPermutation({2, 3, 0, 1});
        // f16 {1, 0, 1, 2}
        const std::vector<uint16_t> vals{0x3C00, 0x0000, 0x3C00, 0x4000};
        const QuantParams q = QuantParams::perTensor(B200C_F16, 0.0039215686274509803, 0, -8, 7);
        auto attr = ContentAttr::get(vals, NDType({1, 4, 1, 1}, B200C_F16)).convertElemType(B200C_SI4).quantCast(q, B200C_SI4).reorder(YXOI);
        NDType resultType({1, 4, 1, 1}, B200C_SI4, q);
        resultType.order = YXOI;
        const DeclareOp op(resultType, attr);
        const DeclareOp folded = foldConstant(be, op);
        const ContentAttr& fa = folded.getContentAttr();
        EXPECT((fa.getBaseType().shape == std::vector<int64_t>{1, 1, 1, 2}) && fa.getBaseType().dtype == B200C_UI8 &&
                       fa.getBaseType().order == YXOI,
               "folded 4-bit constant is stored as 1x1x1x2xui8 in the original order");
        EXPECT(fa.getNumTransformations() == 1 && fa.getTransformationKind(0) == B200C_X_CHANGE_SHAPE_AND_ELEM_TYPE,
               "ChangeShapeAndElemType restores the shape and element type");
        EXPECT((fa.getType().shape == std::vector<int64_t>{1, 4, 1, 1}) && fa.getType().dtype == B200C_SI4, "inferred type is the op's");
        EXPECT((folded.getContent(be).getRawBytes() == std::vector<uint8_t>{16, 18}), "packed bytes [16, 18]");
        std::vector<uint8_t> section{0xAB};
        folded.serialize(be, section);
        EXPECT((section == std::vector<uint8_t>{0xAB, 16, 18}), "serialize appends the constant's bytes");
        // a byte-sized constant folds to an empty transformation list
        std::vector<float> w(24);
        std::iota(w.begin(), w.end(), 0.0f);
        const DeclareOp plain(NDType({2, 3, 2, 2}, B200C_F16, DimsOrder::NHWC()),
                              ContentAttr::get(w, NDType({2, 3, 2, 2}, B200C_F32)).convertElemType(B200C_F16).reorder(DimsOrder::NHWC()));
        const DeclareOp pf = foldConstant(be, plain);
        EXPECT(pf.getContentAttr().getNumTransformations() == 0 && pf.getContentAttr().getBaseType().dtype == B200C_F16,
               "folded constant has an empty list and the folded element type");
        EXPECT(pf.getContent(be).getRawBytes() == plain.getContent(be).getRawBytes(), "folding twice changes nothing");
    }
    // ---- splat detection of a raw buffer (content.cpp:103-137) ----
    {
        std::vector<uint32_t> same(100000, 0xDEADBEEFu), one_off = same;
        one_off[77777] ^= 0x100u;
        EXPECT(detectSplat(be, same.data(), same.size() * 4, 4), "all elements equal");
        EXPECT(!detectSplat(be, one_off.data(), one_off.size() * 4, 4), "one element differs");
        EXPECT(!detectSplat(be, same.data(), 0, 4), "empty data is not a splat");
    }
    // ---- sparsify-weights and the identity filter of a lowered sparsity op (sparsify_weights.cpp:108-164,
    //      lower_sparsity_ops.cpp:209-250) ----
    {
        std::mt19937 rng(11);
        std::vector<int8_t> w(16 * 32);
        for (auto& v : w) v = (rng() % 10 < 4) ? static_cast<int8_t>(static_cast<int>(rng() % 254) - 127) : 0;
        for (auto& v : w)
            if (v == 0 && (rng() % 64) == 0) v = 1;  // keep a few small survivors
        const QuantParams q = QuantParams::perAxis(B200C_F16, std::vector<double>(16, 0.1), std::vector<int64_t>(16, 0), 0, -128, 127);
        const auto base = ContentAttr::get(w, NDType({16, 32, 1, 1}, B200C_SI8)).quantCast(q, B200C_SI8).reorder(DimsOrder::OYXI());
        const chains::SparseWeights sw = chains::sparsifyWeights(be, base);
        EXPECT(sw.values.getNumTransformations() == 2 && sw.values.getTransformationKind(0) == B200C_X_QUANT_CAST &&
                       sw.values.getTransformationKind(1) == B200C_X_SPARSIFY,
               "sparsified weights: a fresh base, QuantCast, Sparsify");
        EXPECT(sw.map.getNumTransformations() == 2 && sw.map.getTransformationKind(1) == B200C_X_GET_SPARSITY_MAP, "sparsity map: QuantCast, GetSparsityMap");
        const auto raw = sw.values.fold(be).getRawBytes();
        const auto map = sw.map.fold(be).getRawBytes();
        bool ok = sw.counts.size() == 16 && map.size() == 16 * 16;
        size_t at = 0;
        for (int oc = 0; ok && oc < 16; ++oc) {
            int64_t n = 0;
            for (int j = 0; j < 32; ++j) {
                const bool nz = w[oc * 32 + j] != 0;
                ok = ok && (((map[oc * 16 + j / 8] >> (j % 8)) & 1) == (nz ? 1 : 0));
                if (nz) {
                    ok = ok && at + n < raw.size() && static_cast<int8_t>(raw[at + n]) == w[oc * 32 + j];
                    ++n;
                }
            }
            ok = ok && sw.counts[oc] == n;
            at += static_cast<size_t>((n + 15) / 16 * 16);
        }
        EXPECT(ok, "sparsify-weights: counts, map bits and compacted runs of a quantised OYXI weight");
        const auto flat = chains::flattenSparseWeights(sw.values, sw.counts);
        EXPECT((flat.getType().shape == std::vector<int64_t>{static_cast<int64_t>(at), 1, 1, 1}), "flattened type holds the aligned runs");
        const auto flatRaw = flat.fold(be).getRawBytes();
        EXPECT(flatRaw.size() >= at && raw.size() >= at && std::memcmp(flatRaw.data(), raw.data(), at) == 0, "flattened content equals the runs");

        const chains::SparseWeights id = chains::sparseIdentityFilter(be, 16, 16, B200C_F16);
        EXPECT((id.counts == std::vector<int64_t>(16, 1)), "identity filter: one survivor per channel");
        const auto idv = id.values.fold(be).getValues<uint16_t>();
        const auto idm = id.map.fold(be).getRawBytes();
        bool idok = idv.size() >= 16 * 8 && idm.size() == 16 * 16;
        for (int oc = 0; idok && oc < 16; ++oc) {
            idok = idv[static_cast<size_t>(oc) * 8] == 0x3C00;  // f16 1.0 at the head of every 16-byte run
            for (int j = 0; idok && j < 16; ++j) idok = (((idm[oc * 16 + j / 8] >> (j % 8)) & 1) == (j == oc ? 1 : 0));
        }
        EXPECT(idok, "identity filter: values and map");
        const QuantParams qi = QuantParams::perTensor(B200C_F16, 1.0, 0, 0, 255);
        const chains::SparseWeights idq = chains::sparseIdentityFilter(be, 16, 16, B200C_UI8, &qi);
        const auto idqv = idq.values.fold(be).getRawBytes();
        bool qok = idq.counts == std::vector<int64_t>(16, 1) && idqv.size() >= 16 * 16;
        for (int oc = 0; qok && oc < 16; ++oc) qok = idqv[static_cast<size_t>(oc) * 16] == 1;
        EXPECT(qok, "quantised identity filter");
    }
    // ---- constant fusion (fuse_constants.cpp:82-176) and the constants-section writers (export.cpp:465-479,
    //      ops.cpp:97-108): the fused bytes are the parts' folded bytes one after the other ----
    {
        std::vector<int32_t> table(4 * 4);
        for (size_t i = 0; i < table.size(); ++i) table[i] = static_cast<int32_t>(1000 + 17 * i);
        std::vector<uint8_t> w(4 * 16);
        for (size_t i = 0; i < w.size(); ++i) w[i] = (i % 3 == 0) ? 0 : static_cast<uint8_t>(i + 1);
        const auto wt = ContentAttr::get(table, NDType({4, 1, 1, 4}, B200C_SI32));
        const auto weights = ContentAttr::get(w, NDType({4, 16, 1, 1}, B200C_UI8)).reorder(DimsOrder::OYXI());
        const auto sm = ContentAttr::get(w, NDType({4, 16, 1, 1}, B200C_UI8)).getSparsityMap();
        auto view = [](int64_t offset, int64_t size) { return std::pair<int64_t, int64_t>(offset, size); };
        const FusedConstant f = fuseConstants(be, &wt, &weights, &sm, nullptr);
        std::vector<uint8_t> want;
        for (const ContentAttr* p : {&wt, &weights, &sm}) {
            const Content c = p->fold(be);
            std::vector<uint8_t> part(static_cast<size_t>(c.getType().getTotalAllocSize()), 0);
            c.copyTo(part.data(), part.size());
            want.insert(want.end(), part.begin(), part.end());
        }
        EXPECT(f.data == want && want.size() == 64 + 64 + 4 * 16, "fused bytes: table, weights, sparsity map");
        EXPECT(f.type.dtype == B200C_UI8 && (f.type.shape == std::vector<int64_t>{1, 1, 1, static_cast<int64_t>(want.size())}), "fused type: [1,1,1,N] ui8");
        EXPECT(f.views.size() == 4 && f.views[0] == view(0, 64) && f.views[1] == view(64, 64) &&
                       f.views[2] == view(128, 64) && f.views[3].first == -1,
               "fused views");
        // f16 weights hold most of the bytes: the fused constant is f16
        std::vector<uint16_t> hw(8 * 16, 0x3C00);
        const auto hweights = ContentAttr::get(hw, NDType({8, 16, 1, 1}, B200C_F16));
        const FusedConstant g = fuseConstants(be, &wt, &hweights, nullptr, nullptr);
        EXPECT(g.type.dtype == B200C_F16 && (g.type.shape == std::vector<int64_t>{1, 1, 1, (64 + 256) / 2}) && g.data.size() == 320, "fused type: f16 majority");
        EXPECT(g.views[0] == view(0, 32) && g.views[1] == view(32, 128) && g.views[2].first == -1,
               "fused views in f16 elements");
        bool tail = true;
        for (size_t i = 64; i < g.data.size(); i += 2) tail = tail && g.data[i] == 0x00 && g.data[i + 1] == 0x3C;
        EXPECT(tail && std::memcmp(g.data.data(), table.data(), 64) == 0, "fused f16 bytes");

        std::vector<uint8_t> five{1, 2, 3, 4, 5};
        std::vector<uint8_t> twelve(12, 9);
        const std::vector<DeclareOp> ops{DeclareOp(NDType({5}, B200C_UI8), ContentAttr::get(five, NDType({5}, B200C_UI8))),
                                         DeclareOp(NDType({12}, B200C_UI8), ContentAttr::get(twelve, NDType({12}, B200C_UI8)))};
        std::vector<size_t> offs;
        const auto schema = writeSection(be, ops, 8, &offs);
        EXPECT(schema.size() == 24 && (offs == std::vector<size_t>{0, 8}) && std::memcmp(schema.data(), five.data(), 5) == 0 && schema[5] == 0 &&
                       schema[7] == 0 && schema[8] == 9 && schema[19] == 9 && schema[20] == 0,
               "graph-schema section: 8-byte aligned, zero padded");
        const auto elf = writeSection(be, ops, 1, &offs);
        EXPECT(elf.size() == 17 && (offs == std::vector<size_t>{0, 5}) && elf[4] == 5 && elf[5] == 9, "ELF section: no padding");
    }
    std::printf("%s\n", failures ? "FAILED" : "OK");
    return failures ? 1 : 0;
}
