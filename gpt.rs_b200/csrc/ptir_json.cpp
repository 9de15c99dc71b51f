// JSON reader + PTIR program model (see ptir_json.h).
#include "ptir_json.h"

#include <cstdio>

#include <cmath>
#include <cstdlib>
#include <cstring>

#include "../../include/gptrs_cuda.h"

namespace gptrs {
namespace ptir {

namespace {

struct Parser {
    const char* p;
    const char* end;
    std::string err;

    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool fail(const char* m) { if (err.empty()) err = m; return false; }

    bool value(Json* out, int depth) {
        if (depth > 64) return fail("json nesting too deep");
        ws();
        if (p >= end) return fail("unexpected end of json");
        char c = *p;
        if (c == '{') {
            ++p; out->kind = Json::Object;
            ws();
            if (p < end && *p == '}') { ++p; return true; }
            for (;;) {
                ws();
                Json key;
                if (p >= end || *p != '"' || !string(&key.str)) return fail("expected object key");
                ws();
                if (p >= end || *p != ':') return fail("expected ':'");
                ++p;
                out->obj.emplace_back(std::move(key.str), Json());
                if (!value(&out->obj.back().second, depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; return true; }
                return fail("expected ',' or '}'");
            }
        }
        if (c == '[') {
            ++p; out->kind = Json::Array;
            ws();
            if (p < end && *p == ']') { ++p; return true; }
            for (;;) {
                out->arr.emplace_back();
                if (!value(&out->arr.back(), depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; return true; }
                return fail("expected ',' or ']'");
            }
        }
        if (c == '"') { out->kind = Json::String; return string(&out->str); }
        if (c == 't' && end - p >= 4 && !strncmp(p, "true", 4)) { p += 4; out->kind = Json::Bool; out->b = true; return true; }
        if (c == 'f' && end - p >= 5 && !strncmp(p, "false", 5)) { p += 5; out->kind = Json::Bool; out->b = false; return true; }
        if (c == 'n' && end - p >= 4 && !strncmp(p, "null", 4)) { p += 4; out->kind = Json::Null; return true; }
        if (c == '-' || (c >= '0' && c <= '9')) {
            char* e = nullptr;
            out->num = strtod(p, &e);
            if (e == p) return fail("bad number");
            p = e; out->kind = Json::Number;
            return true;
        }
        return fail("unexpected character in json");
    }

    bool string(std::string* s) {
        ++p;  // opening quote
        while (p < end && *p != '"') {
            if (*p == '\\') {
                if (p + 1 >= end) return fail("bad escape");
                char e = p[1];
                switch (e) {
                    case 'n': s->push_back('\n'); break;
                    case 't': s->push_back('\t'); break;
                    case 'r': s->push_back('\r'); break;
                    case 'b': s->push_back('\b'); break;
                    case 'f': s->push_back('\f'); break;
                    case 'u': {
                        if (p + 5 >= end) return fail("bad \\u escape");
                        unsigned v = (unsigned)strtoul(std::string(p + 2, 4).c_str(), nullptr, 16);
                        s->push_back(v < 128 ? (char)v : '?');
                        p += 4;
                        break;
                    }
                    default: s->push_back(e);
                }
                p += 2;
            } else {
                s->push_back(*p++);
            }
        }
        if (p >= end) return fail("unterminated string");
        ++p;
        return true;
    }
};

int dtype_of(const std::string& s) {
    if (s == "F32") return GPTRS_F32;
    if (s == "Si32") return GPTRS_SI32;
    if (s == "I1") return GPTRS_I1;
    if (s == "Bf16") return GPTRS_BF16;
    if (s == "F16") return GPTRS_F16;
    if (s == "Si8") return GPTRS_SI8;
    if (s == "Ui8") return GPTRS_UI8;
    return -1;
}

bool read_shape(const Json* shape, std::vector<int64_t>* dims, std::string* err) {
    const Json* d = shape ? shape->get("dims") : nullptr;
    if (!d || d->kind != Json::Array) { *err = "shape without dims"; return false; }
    for (auto& e : d->arr) {
        const Json* st = e.get("Static");
        if (!st) { *err = "dynamic dimensions are not supported at run time"; return false; }
        dims->push_back(st->as_int());
    }
    return true;
}

bool read_tspec(const Json* spec, TSpec* out, std::string* err) {
    if (!spec) { *err = "missing tensor spec"; return false; }
    const Json* dt = spec->get("dtype");
    if (!dt || dt->kind != Json::String) { *err = "tensor spec without dtype"; return false; }
    out->dtype = dtype_of(dt->str);
    if (out->dtype < 0) { *err = "unsupported dtype " + dt->str; return false; }
    return read_shape(spec->get("shape"), &out->dims, err);
}

bool read_value_type(const Json& vt, TSpec* out, std::string* err) {
    const Json* t = vt.get("Tensor");
    if (!t) { *err = "tuple values are not supported"; return false; }
    return read_tspec(t, out, err);
}

// CustomCallAttr is adjacently tagged by serde: {"kind": "F64", "value": 1e-5} (spec.rs:602-613). The externally
// tagged form {"F64": 1e-5} is accepted as well.
const Json* attr_value(const Json* a, const char* kind) {
    if (!a || a->kind != Json::Object) return nullptr;
    const Json* k = a->get("kind");
    if (k && k->kind == Json::String && k->str == kind) return a->get("value");
    return a->get(kind);
}

void read_ints(const Json* a, std::vector<int64_t>* out) {
    if (!a) return;
    for (auto& e : a->arr) out->push_back(e.as_int());
}

}  // namespace

bool parse_json(const char* text, size_t len, Json* out, std::string* err) {
    Parser ps{text, text + len, {}};
    if (!ps.value(out, 0)) { *err = ps.err; return false; }
    ps.ws();
    if (ps.p != ps.end) { *err = "trailing characters after json"; return false; }
    return true;
}

void write_json(const Json& j, std::string* out) {
    switch (j.kind) {
        case Json::Null: *out += "null"; break;
        case Json::Bool: *out += j.b ? "true" : "false"; break;
        case Json::Number: {
            char buf[40];
            if (j.num == (double)(int64_t)j.num && j.num > -9.0e15 && j.num < 9.0e15) snprintf(buf, sizeof buf, "%lld", (long long)j.num);
            else snprintf(buf, sizeof buf, "%.17g", j.num);
            *out += buf;
            break;
        }
        case Json::String: {
            *out += '"';
            for (unsigned char c : j.str) {
                if (c == '"' || c == '\\') { *out += '\\'; *out += (char)c; }
                else if (c < 0x20) { char buf[8]; snprintf(buf, sizeof buf, "\\u%04x", c); *out += buf; }
                else *out += (char)c;
            }
            *out += '"';
            break;
        }
        case Json::Array:
            *out += '[';
            for (size_t i = 0; i < j.arr.size(); ++i) { if (i) *out += ','; write_json(j.arr[i], out); }
            *out += ']';
            break;
        case Json::Object:
            *out += '{';
            for (size_t i = 0; i < j.obj.size(); ++i) {
                if (i) *out += ',';
                Json k; k.kind = Json::String; k.str = j.obj[i].first;
                write_json(k, out);
                *out += ':';
                write_json(j.obj[i].second, out);
            }
            *out += '}';
            break;
    }
}

const char* fused_target(Op op) {
    switch (op) {
        case Op::FusedLayerNorm: return "gpt_rs.cuda.layer_norm.f32.v1";
        case Op::FusedRmsNorm: return "gpt_rs.cuda.rms_norm.f32.v1";
        case Op::FusedSoftmax: return "gpt_rs.cuda.softmax_last_axis.f32.v1";
        case Op::FusedMatmulBias: return "gpt_rs.cuda.matmul_bias.f32.v1";
        case Op::FusedAttentionDecode: return "gpt_rs.cuda.attention_decode.f32.v1";
        case Op::FusedAddRmsNorm: return "gpt_rs.cuda.add_rms_norm.f32.v1";
        case Op::FusedAddLayerNorm: return "gpt_rs.cuda.add_layer_norm.f32.v1";
        case Op::FusedGelu: return "gpt_rs.cuda.gelu.f32.v1";
        default: return nullptr;
    }
}

int build_function(const Json& program, Function* fn, std::string* err) {
    const Json* ver = program.get("spec_version");
    if (ver && ver->str != "ptir.v0.4") { *err = "unsupported PTIR spec version '" + ver->str + "'"; return 1; }
    const Json* entry = program.get("entry");
    const Json* fns = program.get("functions");
    if (!entry || !fns) { *err = "program without entry/functions"; return 1; }
    const Json* f = nullptr;
    for (auto& cand : fns->arr) {
        const Json* n = cand.get("name");
        if (n && n->str == entry->str) f = &cand;
    }
    if (!f) { *err = "entry function not found"; return 1; }
    const Json *params = f->get("parameters"), *pids = f->get("parameter_ids"), *body = f->get("body"),
               *rids = f->get("result_ids");
    if (!params || !pids || !body || !rids || params->arr.size() != pids->arr.size()) { *err = "malformed function"; return 1; }
    for (size_t i = 0; i < params->arr.size(); ++i) {
        TSpec t;
        if (!read_value_type(params->arr[i], &t, err)) return 1;
        fn->params.push_back(t);
        fn->param_ids.push_back((uint32_t)pids->arr[i].as_int());
    }
    for (auto& r : rids->arr) fn->result_ids.push_back((uint32_t)r.as_int());
    for (auto& ji : body->arr) {
        Inst in;
        const Json *id = ji.get("id"), *op = ji.get("op"), *ops = ji.get("operands"), *outp = ji.get("output");
        if (!id || !op || !ops || !outp) { *err = "malformed instruction"; return 1; }
        in.id = (uint32_t)id->as_int();
        if (!read_value_type(*outp, &in.out, err)) return 1;
        for (auto& jo : ops->arr) {
            Operand o;
            if (const Json* v = jo.get("Value")) {
                o.id = (uint32_t)v->as_int();
            } else if (const Json* l = jo.get("Literal")) {
                o.is_literal = true;
                if (!read_tspec(l->get("spec"), &o.lit, err)) return 1;
                const Json* by = l->get("bytes");
                if (!by) { *err = "literal without bytes"; return 1; }
                for (auto& e : by->arr) o.bytes.push_back((uint8_t)e.as_int());
            } else {
                *err = "tuple operands are not supported";
                return 2;
            }
            in.operands.push_back(std::move(o));
        }
        const Json* attr = nullptr;
        if (op->kind == Json::String) {
            in.name = op->str;
        } else if (op->kind == Json::Object && op->obj.size() == 1) {
            in.name = op->obj[0].first;
            attr = &op->obj[0].second;
        } else {
            *err = "malformed operation";
            return 1;
        }
        const std::string& n = in.name;
        static const char* const kNeedsAttr[] = {"Constant", "ElementwiseUnary", "ElementwiseBinary", "DotGeneral", "Reduce", "Compare", "Cast",
                                                 "Transpose", "Slice", "Concat", "Iota", "Gather", "DynamicSlice", "DynamicUpdateSlice",
                                                 "ReduceWindow", "CustomCall", "Dequantize"};
        for (const char* k : kNeedsAttr)
            if (n == k && !attr) { *err = n + " (%" + std::to_string(in.id) + ") without its attributes"; return 1; }
        if ((n == "ElementwiseUnary" || n == "ElementwiseBinary") && attr->kind != Json::String) { *err = n + ": the operation kind must be a string"; return 1; }
        if (n != "ElementwiseUnary" && n != "ElementwiseBinary" && attr && attr->kind != Json::Object) { *err = n + ": attributes must be an object"; return 1; }
        if (n == "Constant") {
            in.op = Op::Constant;
            Operand o; o.is_literal = true;
            if (!read_tspec(attr->get("spec"), &o.lit, err)) return 1;
            if (const Json* by = attr->get("bytes")) for (auto& e : by->arr) o.bytes.push_back((uint8_t)e.as_int());
            in.operands.push_back(std::move(o));
        } else if (n == "ElementwiseUnary") { in.op = Op::Unary; in.sub = attr->str; }
        else if (n == "ElementwiseBinary") { in.op = Op::Binary; in.sub = attr->str; }
        else if (n == "DotGeneral") {
            in.op = Op::DotGeneral;
            read_ints(attr->get("batch_lhs"), &in.a); read_ints(attr->get("batch_rhs"), &in.b);
            read_ints(attr->get("contract_lhs"), &in.c); read_ints(attr->get("contract_rhs"), &in.d);
        } else if (n == "Reduce") {
            in.op = Op::Reduce;
            in.sub = attr->get("kind") ? attr->get("kind")->str : "";
            read_ints(attr->get("axes"), &in.a);
            in.keepdims = attr->get("keepdims") && attr->get("keepdims")->b;
        } else if (n == "Compare") { in.op = Op::Compare; in.sub = attr->get("op") ? attr->get("op")->str : ""; }
        else if (n == "Select") in.op = Op::Select;
        else if (n == "Cast") { in.op = Op::Cast; in.sub = attr->get("dtype") ? attr->get("dtype")->str : ""; }
        else if (n == "StopGradient") in.op = Op::StopGradient;
        else if (n == "Reshape") in.op = Op::Reshape;
        else if (n == "Transpose") { in.op = Op::Transpose; read_ints(attr->get("perm"), &in.a); }
        else if (n == "BroadcastTo") in.op = Op::BroadcastTo;
        else if (n == "Slice") { in.op = Op::Slice; read_ints(attr->get("starts"), &in.a); read_ints(attr->get("sizes"), &in.b); }
        else if (n == "Concat") { in.op = Op::Concat; in.axis = attr->get("axis") ? attr->get("axis")->as_int() : 0; }
        else if (n == "Iota") { in.op = Op::Iota; in.axis = attr->get("axis") ? attr->get("axis")->as_int() : 0; }
        else if (n == "Take") in.op = Op::Take;
        else if (n == "Gather") { in.op = Op::Gather; in.axis = attr->get("axis") ? attr->get("axis")->as_int() : 0; }
        else if (n == "DynamicSlice") { in.op = Op::DynamicSlice; read_ints(attr->get("sizes"), &in.a); }
        else if (n == "DynamicUpdateSlice") { in.op = Op::DynamicUpdateSlice; read_ints(attr->get("sizes"), &in.a); }
        else if (n == "ReduceWindow") {
            // ReduceWindowSpec (spec.rs:532-543): a = window, b = strides, c = low padding, d = base dilation, e = window dilation
            in.op = Op::ReduceWindow;
            in.sub = attr->get("reduce") ? attr->get("reduce")->str : "";
            read_ints(attr->get("window_dims"), &in.a); read_ints(attr->get("strides"), &in.b);
            if (const Json* pad = attr->get("padding"))
                for (auto& pr : pad->arr) in.c.push_back(pr.arr.empty() ? 0 : pr.arr[0].as_int());
            read_ints(attr->get("base_dilation"), &in.d); read_ints(attr->get("window_dilation"), &in.e);
            const Json* acc = attr->get("accum_dtype");
            if (acc && acc->kind == Json::String && acc->str != "F32") in.f0 = 1.f;  // refused at run time like the reference
        }
        else if (n == "Dequantize") {
            // DequantizeSpec { axis, output_dtype } (spec.rs:585-589). The scheme is backend-defined (docs/backend.md:620-632);
            // this backend's: (q si8 [N][K], fp16 scales [N]) or (q ui8 [N][K/2] = two si4 per byte, low nibble first,
            // fp16 scales [N][K/128]) -> f32 [N][K], w = q * scale.
            in.op = Op::Dequantize;
        }
        else if (n == "CustomCall") {
            in.op = Op::CustomCall;
            in.sub = attr->get("target") ? attr->get("target")->str : "";
            // the targets written by this backend's own fusion pipeline come back as the fused operations
            const Json* attrs = attr->get("attrs");
            if (in.sub == "gpt_rs.cuda.quant_matmul_w4a16.v1" || in.sub == "gpt_rs.cuda.quant_matmul_w8a16.v1") {
                if (in.operands.size() != 3) { *err = in.sub + ": wrong operand count"; return 1; }
                in.op = Op::FusedQuantMatmul;
                in.sub = in.sub == "gpt_rs.cuda.quant_matmul_w8a16.v1" ? "w8" : "w4";
            }
            for (Op f : {Op::FusedLayerNorm, Op::FusedRmsNorm, Op::FusedSoftmax, Op::FusedMatmulBias, Op::FusedAttentionDecode, Op::FusedAddRmsNorm,
                         Op::FusedAddLayerNorm, Op::FusedGelu}) {
                if (in.op != Op::CustomCall || in.sub != fused_target(f)) continue;
                const size_t want = f == Op::FusedLayerNorm || f == Op::FusedMatmulBias || f == Op::FusedAddRmsNorm ? 3
                                    : f == Op::FusedRmsNorm ? 2 : (f == Op::FusedSoftmax || f == Op::FusedGelu) ? 1 : 4;
                if (in.operands.size() != want) { *err = in.sub + ": wrong operand count"; return 1; }
                in.op = f;
                if (f == Op::FusedLayerNorm || f == Op::FusedRmsNorm || f == Op::FusedAddRmsNorm || f == Op::FusedAddLayerNorm) {
                    const Json* e = attrs ? attrs->get("eps") : nullptr;
                    const Json* v = attr_value(e, "F64");
                    if (!v || v->kind != Json::Number) { *err = in.sub + ": attribute eps (F64) is required"; return 1; }
                    in.f0 = (float)v->num;
                }
                if (f == Op::FusedMatmulBias) {   // optional: the activation applied to the sum ("gelu")
                    const Json* a = attrs ? attrs->get("activation") : nullptr;
                    const Json* v = attr_value(a, "String");
                    if (v && v->kind == Json::String) {
                        if (v->str != "gelu") { *err = in.sub + ": unknown activation '" + v->str + "'"; return 1; }
                        in.axis = 1;
                    }
                }
                if (f == Op::FusedAttentionDecode) {
                    const Json* g = attrs ? attrs->get("geometry") : nullptr;
                    read_ints(attr_value(g, "I64Array"), &in.a);
                    if (in.a.size() != 4) { *err = in.sub + ": attribute geometry (I64Array of q heads, kv heads, head_dim, capacity) is required"; return 1; }
                }
            }
        }
        else in.op = Op::Unsupported;
        in.src = (int)fn->body.size();
        fn->body.push_back(std::move(in));
    }
    return 0;
}

}  // namespace ptir
}  // namespace gptrs
