// Structural verification of a parsed PTIR function before anything is launched: operand counts, attribute
// ranges and the declared result type of every instruction against the type its operands imply. The reference
// interpreter rejects a malformed program with an error (crates/gpt-rs-backend-ref-cpu/src/cpu.rs validates the
// operands of every instruction it executes); here the same checks run once per plan, on the host, so that a
// mismatched program can never turn into an out-of-bounds access on the device.
#include <algorithm>
#include <unordered_map>

#include "../../include/gptrs_cuda.h"
#include "ptir_json.h"

namespace gptrs {
namespace ptir {
namespace {

size_t elem_size(int dtype) {
    switch (dtype) {
        case GPTRS_F32: case GPTRS_SI32: return 4;
        case GPTRS_F16: case GPTRS_BF16: return 2;
        case GPTRS_I1: case GPTRS_SI8: case GPTRS_UI8: return 1;
        default: return 0;
    }
}

std::string dims_text(const std::vector<int64_t>& d) {
    std::string s = "[";
    for (size_t i = 0; i < d.size(); ++i) s += (i ? "," : "") + std::to_string(d[i]);
    return s + "]";
}

bool in_range_unique(const std::vector<int64_t>& axes, int64_t rank) {
    std::vector<bool> seen((size_t)std::max<int64_t>(rank, 0), false);
    for (int64_t a : axes) {
        if (a < 0 || a >= rank || seen[(size_t)a]) return false;
        seen[(size_t)a] = true;
    }
    return true;
}

}  // namespace

int verify_function(const Function& fn, std::string* err) {
    std::unordered_map<uint32_t, const TSpec*> types;
    for (size_t i = 0; i < fn.param_ids.size(); ++i) {
        if (!types.emplace(fn.param_ids[i], &fn.params[i]).second) { *err = "duplicate parameter id %" + std::to_string(fn.param_ids[i]); return 1; }
        for (int64_t d : fn.params[i].dims) if (d < 0) { *err = "negative dimension in a parameter type"; return 1; }
    }
    for (const Inst& in : fn.body) {
        auto bad = [&](const std::string& why) {
            *err = in.name + " (%" + std::to_string(in.id) + "): " + why;
            return 1;
        };
        if (in.dead) continue;
        for (int64_t d : in.out.dims) if (d < 0) return bad("negative dimension in the declared output");
        if (in.out.dims.size() > 8) return bad("rank above 8");
        // operand types
        std::vector<const TSpec*> s;
        for (const Operand& o : in.operands) {
            if (o.is_literal) {
                for (int64_t d : o.lit.dims) if (d < 0) return bad("negative dimension in a literal");
                if (o.bytes.size() != (size_t)o.lit.numel() * elem_size(o.lit.dtype)) return bad("literal byte length does not match its type");
                s.push_back(&o.lit);
            } else {
                auto it = types.find(o.id);
                if (it == types.end()) return bad("use of undefined value %" + std::to_string(o.id));
                s.push_back(it->second);
            }
        }
        const TSpec& O = in.out;
        const size_t n = s.size();
        auto arity = [&](size_t want) { return n == want; };
        auto same = [](const TSpec& a, const TSpec& b) { return a.dtype == b.dtype && a.dims == b.dims; };
        auto expect_out = [&](int dtype, const std::vector<int64_t>& dims) -> int {
            if (O.dtype != dtype || O.dims != dims) return bad("declared output " + dims_text(O.dims) + " does not match the operands (" + dims_text(dims) + ")");
            return 0;
        };
        int rc = 0;
        switch (in.op) {
            case Op::Constant:
                if (!arity(1) || !in.operands[0].is_literal) return bad("constant without a literal");
                rc = expect_out(s[0]->dtype, s[0]->dims);
                break;
            case Op::Unary: case Op::StopGradient:
                if (!arity(1)) return bad("expects 1 operand");
                rc = expect_out(s[0]->dtype, s[0]->dims);
                break;
            case Op::Binary:
                if (!arity(2)) return bad("expects 2 operands");
                if (!same(*s[0], *s[1])) return bad("operand shapes or dtypes differ");
                rc = expect_out(s[0]->dtype, s[0]->dims);
                break;
            case Op::Compare:
                if (!arity(2)) return bad("expects 2 operands");
                if (!same(*s[0], *s[1])) return bad("operand shapes or dtypes differ");
                rc = expect_out(GPTRS_I1, s[0]->dims);
                break;
            case Op::Select:
                if (!arity(3)) return bad("expects 3 operands");
                if (s[0]->dtype != GPTRS_I1 || !same(*s[1], *s[2]) || s[0]->dims != s[1]->dims) return bad("select needs an i1 predicate and equal branches of its shape");
                rc = expect_out(s[1]->dtype, s[1]->dims);
                break;
            case Op::Cast:
                if (!arity(1)) return bad("expects 1 operand");
                if (O.dims != s[0]->dims) return bad("cast changes the shape");
                break;
            case Op::Reshape:
                if (!arity(1)) return bad("expects 1 operand");
                if (O.dtype != s[0]->dtype || O.numel() != s[0]->numel()) return bad("element count or dtype changes");
                break;
            case Op::Transpose: {
                if (!arity(1)) return bad("expects 1 operand");
                const int64_t r = (int64_t)s[0]->dims.size();
                if ((int64_t)in.a.size() != r || !in_range_unique(in.a, r)) return bad("perm is not a permutation of the operand's axes");
                std::vector<int64_t> d((size_t)r);
                for (int64_t i = 0; i < r; ++i) d[(size_t)i] = s[0]->dims[(size_t)in.a[(size_t)i]];
                rc = expect_out(s[0]->dtype, d);
                break;
            }
            case Op::BroadcastTo: {
                if (!arity(1)) return bad("expects 1 operand");
                if (s[0]->dims.size() > O.dims.size() || O.dtype != s[0]->dtype) return bad("operand rank above the output rank, or dtype changes");
                const size_t shift = O.dims.size() - s[0]->dims.size();
                for (size_t d = 0; d < s[0]->dims.size(); ++d)
                    if (s[0]->dims[d] != 1 && s[0]->dims[d] != O.dims[d + shift]) return bad("shapes are not broadcast compatible");
                break;
            }
            case Op::Slice: {
                if (!arity(1)) return bad("expects 1 operand");
                const size_t r = s[0]->dims.size();
                if (in.a.size() != r || in.b.size() != r) return bad("starts / sizes must have one entry per axis");
                for (size_t d = 0; d < r; ++d)
                    if (in.a[d] < 0 || in.b[d] < 0 || in.a[d] + in.b[d] > s[0]->dims[d]) return bad("slice out of bounds");
                rc = expect_out(s[0]->dtype, in.b);
                break;
            }
            case Op::Concat: {
                if (n == 0) return bad("expects at least 1 operand");
                const int64_t r = (int64_t)s[0]->dims.size();
                const int64_t ax = in.axis < 0 ? in.axis + r : in.axis;
                if (ax < 0 || ax >= r) return bad("axis out of range");
                std::vector<int64_t> d = s[0]->dims;
                d[(size_t)ax] = 0;
                for (const TSpec* t : s) {
                    if (t->dtype != s[0]->dtype || (int64_t)t->dims.size() != r) return bad("operands differ in dtype or rank");
                    for (int64_t i = 0; i < r; ++i)
                        if (i != ax && t->dims[(size_t)i] != s[0]->dims[(size_t)i]) return bad("operands differ outside the concat axis");
                    d[(size_t)ax] += t->dims[(size_t)ax];
                }
                rc = expect_out(s[0]->dtype, d);
                break;
            }
            case Op::Iota:
                if (!arity(0)) return bad("expects no operand");
                if (in.axis < 0 || in.axis >= (int64_t)O.dims.size()) return bad("axis out of range");
                break;
            case Op::Take: {
                if (!arity(2)) return bad("expects 2 operands");
                if (s[0]->dims.empty() || s[1]->dtype != GPTRS_SI32) return bad("take needs a table of rank >= 1 and si32 indices");
                std::vector<int64_t> d = s[1]->dims;
                d.insert(d.end(), s[0]->dims.begin() + 1, s[0]->dims.end());
                rc = expect_out(s[0]->dtype, d);
                break;
            }
            case Op::Gather: {
                if (!arity(2)) return bad("expects 2 operands");
                const int64_t r = (int64_t)s[0]->dims.size();
                const int64_t ax = in.axis < 0 ? in.axis + r : in.axis;
                if (ax < 0 || ax >= r || s[1]->dtype != GPTRS_SI32 || (int64_t)s[1]->dims.size() != r) return bad("axis out of range, or indices of another rank / dtype");
                for (int64_t i = 0; i < r; ++i)
                    if (i != ax && s[1]->dims[(size_t)i] != s[0]->dims[(size_t)i]) return bad("indices differ from the operand outside the gather axis");
                rc = expect_out(s[0]->dtype, s[1]->dims);
                break;
            }
            case Op::DynamicSlice: {
                if (!arity(2)) return bad("expects 2 operands");
                const size_t r = s[0]->dims.size();
                if (in.a.size() != r || s[1]->dtype != GPTRS_SI32 || s[1]->numel() != (int64_t)r) return bad("sizes / starts must have one entry per axis (starts si32)");
                for (size_t d = 0; d < r; ++d)
                    if (in.a[d] < 0 || in.a[d] > s[0]->dims[d]) return bad("slice larger than the operand");
                rc = expect_out(s[0]->dtype, in.a);
                break;
            }
            case Op::DynamicUpdateSlice: {
                if (!arity(3)) return bad("expects 3 operands");
                const size_t r = s[0]->dims.size();
                if (s[1]->dims.size() != r || s[1]->dtype != s[0]->dtype || s[2]->dtype != GPTRS_SI32 || s[2]->numel() != (int64_t)r)
                    return bad("update must have the operand's rank and dtype, starts si32[rank]");
                for (size_t d = 0; d < r; ++d)
                    if (s[1]->dims[d] > s[0]->dims[d]) return bad("update larger than the operand");
                rc = expect_out(s[0]->dtype, s[0]->dims);
                break;
            }
            case Op::Reduce: {
                if (!arity(1)) return bad("expects 1 operand");
                const int64_t r = (int64_t)s[0]->dims.size();
                if (in.a.empty() || !in_range_unique(in.a, r)) return bad("axes out of range or repeated");
                std::vector<int64_t> d;
                for (int64_t i = 0; i < r; ++i) {
                    const bool red = std::find(in.a.begin(), in.a.end(), i) != in.a.end();
                    if (!red) d.push_back(s[0]->dims[(size_t)i]);
                    else if (in.keepdims) d.push_back(1);
                }
                if (O.dims != d) return bad("declared output " + dims_text(O.dims) + " is not the reduced shape " + dims_text(d));
                break;
            }
            case Op::DotGeneral: {
                if (!arity(2)) return bad("expects 2 operands");
                const int64_t ra = (int64_t)s[0]->dims.size(), rb = (int64_t)s[1]->dims.size();
                std::vector<int64_t> la = in.a, lb = in.b;
                la.insert(la.end(), in.c.begin(), in.c.end());
                lb.insert(lb.end(), in.d.begin(), in.d.end());
                if (in.a.size() != in.b.size() || in.c.size() != in.d.size() || !in_range_unique(la, ra) || !in_range_unique(lb, rb))
                    return bad("batch / contracting axes out of range, repeated or of different counts");
                std::vector<int64_t> d;
                for (size_t i = 0; i < in.a.size(); ++i) {
                    if (s[0]->dims[(size_t)in.a[i]] != s[1]->dims[(size_t)in.b[i]]) return bad("batch sizes differ");
                    d.push_back(s[0]->dims[(size_t)in.a[i]]);
                }
                for (size_t i = 0; i < in.c.size(); ++i)
                    if (s[0]->dims[(size_t)in.c[i]] != s[1]->dims[(size_t)in.d[i]]) return bad("contracting sizes differ");
                for (int64_t i = 0; i < ra; ++i) if (std::find(la.begin(), la.end(), i) == la.end()) d.push_back(s[0]->dims[(size_t)i]);
                for (int64_t i = 0; i < rb; ++i) if (std::find(lb.begin(), lb.end(), i) == lb.end()) d.push_back(s[1]->dims[(size_t)i]);
                if (O.dims != d) return bad("declared output " + dims_text(O.dims) + " is not the contraction's shape " + dims_text(d));
                break;
            }
            case Op::ReduceWindow:
                if (!arity(1)) return bad("expects 1 operand");
                break;
            case Op::Dequantize: {
                // (q si8 [N][K], scales f16 [N]) or (q ui8 [N][K/2] holding two si4, scales f16 [N][K/128]) -> f32 [N][K]
                if (!arity(2)) return bad("expects 2 operands (quantised values, fp16 scales)");
                if (s[0]->dims.size() != 2 || s[1]->dtype != GPTRS_F16 || O.dtype != GPTRS_F32 || O.dims.size() != 2) return bad("rank-2 quantised values, fp16 scales and an f32 result are expected");
                const int64_t rows = s[0]->dims[0];
                if (s[0]->dtype == GPTRS_SI8) {
                    if (s[1]->dims != std::vector<int64_t>{rows} || O.dims != s[0]->dims) return bad("si8 values need one scale per row and a result of their shape");
                } else if (s[0]->dtype == GPTRS_UI8) {
                    const int64_t k = s[0]->dims[1] * 2;
                    if (k % 128 != 0 || s[1]->dims != std::vector<int64_t>{rows, k / 128} || O.dims != std::vector<int64_t>{rows, k})
                        return bad("packed si4 values [N][K/2] need scales [N][K/128] and a result [N][K], K a multiple of 128");
                } else return bad("quantised values must be si8 or ui8 (two packed si4)");
                break;
            }
            case Op::FusedLayerNorm: case Op::FusedRmsNorm: case Op::FusedAddRmsNorm: case Op::FusedAddLayerNorm: {
                const bool add = in.op == Op::FusedAddRmsNorm || in.op == Op::FusedAddLayerNorm;
                const bool ln = in.op == Op::FusedLayerNorm || in.op == Op::FusedAddLayerNorm;
                const size_t want = (add ? 2 : 1) + (ln ? 2 : 1);
                if (!arity(want)) return bad("wrong operand count");
                if (s[0]->dims.empty() || s[0]->dtype != GPTRS_F32) return bad("f32 rows expected");
                const std::vector<int64_t> row = {s[0]->dims.back()};
                if (add && !same(*s[0], *s[1])) return bad("residual and update differ");
                for (size_t i = add ? 2 : 1; i < want; ++i)
                    if (s[i]->dtype != GPTRS_F32 || s[i]->dims != row) return bad("gain / shift must be f32 [row width]");
                rc = expect_out(GPTRS_F32, s[0]->dims);
                break;
            }
            case Op::FusedGelu:
            case Op::FusedSoftmax:
                if (!arity(1)) return bad("wrong operand count");
                if (s[0]->dims.empty() || s[0]->dtype != GPTRS_F32) return bad("f32 rows expected");
                rc = expect_out(GPTRS_F32, s[0]->dims);
                break;
            case Op::FusedMatmulBias: {
                if (!arity(3)) return bad("wrong operand count");
                if (s[0]->dims.size() != 2 || s[1]->dims.size() != 2 || s[0]->dims[1] != s[1]->dims[0] || s[2]->dims != std::vector<int64_t>{s[1]->dims[1]} ||
                    s[0]->dtype != GPTRS_F32 || s[1]->dtype != GPTRS_F32 || s[2]->dtype != GPTRS_F32)
                    return bad("x [M,K], w [K,N] and bias [N] (f32) expected");
                rc = expect_out(GPTRS_F32, {s[0]->dims[0], s[1]->dims[1]});
                break;
            }
            case Op::FusedQuantMatmul: {
                // (x f32 [M][K], q, scales) -> f32 [M][N]; q / scales as for Dequantize
                if (!arity(3)) return bad("wrong operand count");
                if (s[0]->dims.size() != 2 || s[0]->dtype != GPTRS_F32 || s[1]->dims.size() != 2 || s[2]->dtype != GPTRS_F16) return bad("x f32 [M,K], rank-2 quantised values and fp16 scales expected");
                const int64_t k = s[0]->dims[1], rows = s[1]->dims[0];
                if (k % 128 != 0 || rows % 16 != 0) return bad("K must be a multiple of 128 and N of 16");
                if (s[1]->dtype == GPTRS_SI8) {
                    if (s[1]->dims[1] != k || s[2]->dims != std::vector<int64_t>{rows}) return bad("si8 weights [N][K] with scales [N] expected");
                } else if (s[1]->dtype == GPTRS_UI8) {
                    if (s[1]->dims[1] * 2 != k || s[2]->dims != std::vector<int64_t>{rows, k / 128}) return bad("packed si4 weights [N][K/2] with scales [N][K/128] expected");
                } else return bad("quantised values must be si8 or ui8 (two packed si4)");
                rc = expect_out(GPTRS_F32, {s[0]->dims[0], rows});
                break;
            }
            case Op::FusedAttentionDecode: {
                if (!arity(4) || in.a.size() != 4) return bad("wrong operand count or geometry");
                const int64_t hq = in.a[0], hkv = in.a[1], hd = in.a[2], cap = in.a[3];
                if (hq <= 0 || hkv <= 0 || hq % hkv != 0 || hd <= 0 || hd > 128 || cap <= 0 || cap > 32768) return bad("geometry out of range");
                if (s[0]->dtype != GPTRS_F32 || s[0]->dims != std::vector<int64_t>{hq, 1, hd} || s[1]->dtype != GPTRS_F32 || s[2]->dtype != GPTRS_F32 ||
                    s[1]->dims != std::vector<int64_t>{hkv, cap, hd} || s[2]->dims != s[1]->dims || s[3]->dtype != GPTRS_SI32 || s[3]->numel() != 1)
                    return bad("q [Hq,1,hd], caches [Hkv,cap,hd] (f32) and a si32 start expected");
                rc = expect_out(GPTRS_F32, s[0]->dims);
                break;
            }
            default:
                break;  // CustomCall with a foreign target and operations outside the subset are refused when executed
        }
        if (rc) return rc;
        if (!types.emplace(in.id, &in.out).second) return bad("value id defined twice");
    }
    for (uint32_t r : fn.result_ids)
        if (!types.count(r)) { *err = "result %" + std::to_string(r) + " is undefined"; return 1; }
    return 0;
}

}  // namespace ptir
}  // namespace gptrs
