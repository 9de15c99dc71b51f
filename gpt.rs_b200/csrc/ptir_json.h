// Minimal JSON reader and the PTIR program model for `run_program`
// (serde wire form of crates/gpt-rs/src/backend/spec.rs:644-756: externally tagged enums,
// `TensorLiteral.bytes` as an array of numbers, `ValueId` as a bare number).
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace gptrs {
namespace ptir {

struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;
    const Json* get(const char* key) const {
        for (auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    int64_t as_int() const { return (int64_t)num; }
};

// Returns false and fills `err` on malformed input.
bool parse_json(const char* text, size_t len, Json* out, std::string* err);
// Compact text of a tree (numbers that hold an integer are written without a fraction).
void write_json(const Json& j, std::string* out);

enum class Op {
    Constant, Unary, Binary, DotGeneral, Reduce, Compare, Select, Cast, StopGradient, Reshape, Transpose, BroadcastTo,
    Slice, Concat, Iota, Take, Gather, DynamicSlice, DynamicUpdateSlice, ReduceWindow, Dequantize, CustomCall,
    // produced by the fusion rewrites of this backend
    FusedLayerNorm, FusedRmsNorm, FusedSoftmax, FusedMatmulBias, FusedAttentionDecode, FusedAddRmsNorm, FusedAddLayerNorm,
    FusedQuantMatmul, FusedGelu, Unsupported
};

struct TSpec {
    int dtype = 0;  // gptrs_dtype
    std::vector<int64_t> dims;
    int64_t numel() const { int64_t n = 1; for (auto d : dims) n *= d; return n; }
};

struct Operand {
    bool is_literal = false;
    uint32_t id = 0;
    TSpec lit;
    std::vector<uint8_t> bytes;
    void* device = nullptr;  // literal uploaded once when the plan is built (a retained Tensor*)
};

struct Inst {
    uint32_t id = 0;
    Op op = Op::Unsupported;
    std::string name;             // operation name as written (for error messages)
    std::string sub;              // unary / binary / compare / reduce kind, cast dtype, custom target
    std::vector<int64_t> a, b, c, d, e;  // attribute vectors (meaning depends on op)
    int64_t axis = 0;
    bool keepdims = false;
    float f0 = 0.f;               // fused ops: eps
    std::vector<Operand> operands;
    TSpec out;
    bool dead = false;            // removed by a rewrite
    int src = -1;                 // index of the instruction in the function body it was read from
    // A fused residual-add + norm also produces the sum itself when other instructions read it: the value id and type
    // of that second result (0 = none). Only the in-process rewrite uses it; the CustomCall text form has one result.
    uint32_t side_id = 0;
    TSpec side_out;
};

struct Function {
    std::vector<uint32_t> param_ids, result_ids;
    std::vector<TSpec> params;
    std::vector<Inst> body;
};

// Builds the entry function. status: 0 ok, 1 spec violation, 2 unimplemented.
int build_function(const Json& program, Function* fn, std::string* err);

// Checks operand counts, attribute ranges and every declared result type against the operand types
// (ptir_verify.cpp). status: 0 ok, 1 spec violation.
int verify_function(const Function& fn, std::string* err);

// CustomCall targets the fusion pipeline of this backend emits and run_program accepts (docs/backend.md:568-592:
// namespaced and versioned).
const char* fused_target(Op op);

}  // namespace ptir
}  // namespace gptrs
