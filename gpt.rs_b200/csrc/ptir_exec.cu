// PortableBackend::run_program for PTIR (ptir.v0.4) programs
// (crates/gpt-rs/src/backend/spec.rs:1325-1329; callers: GraphArena::try_execute_plan,
// crates/gpt-rs/src/ops/graph/arena.rs:1014).
//
// A program arrives as serde JSON (`Program::to_json_string`, spec.rs:799-817). It is parsed once,
// rewritten (norm / softmax / matmul+bias subgraphs -> fused kernels, the C++ counterpart of the
// `#[ptir_pattern]` rewrites a backend installs in its pipeline's `pre` phase,
// crates/gpt-rs/src/backend/pipeline.rs:60-119) and cached by a hash of the text: the arena re-sends the
// byte-identical program every decode step. Execution walks the instruction list; every operation
// is one kernel launch on device tensors (f32 / si32 / i1), no host round trips:
// DynamicSlice / DynamicUpdateSlice read their start indices on the device and clamp them there
// (docs/backend.md:452-474).
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "ptir_json.h"
#include "tensor.h"

namespace gptrs {

// norm_embed_sample.cu: out = norm(hidden_in + delta) with the sum optionally written to sum_out (any of the three row
// buffers may be the same memory); layer_norm selects LayerNorm (beta may be null) or RMSNorm.
int add_norm_out_of_place(const float* hidden_in, const float* delta, float* sum_out, const float* gamma, const float* beta, float eps,
                          float* out, int64_t rows, int64_t dim, bool layer_norm, cudaStream_t st);

namespace ptir {
namespace {

constexpr int kMaxRank = 8;

// ---- generic strided copy: out[o_off + idx . o_str] = in[i_off + idx . i_str] over `dims` -------
struct CopyParams {
    const void* in;
    void* out;
    int rank;
    int64_t dims[kMaxRank], i_str[kMaxRank], o_str[kMaxRank];
    int64_t i_off, o_off, n;
    // dynamic offsets: starts[d] (si32, device) clamped into [0, limit[d]] scales dyn_str[d]
    const int* starts;
    int dyn_rank;
    int64_t dyn_limit[kMaxRank], dyn_str[kMaxRank];
    int dyn_on_out;
};

template <typename T>
__global__ void strided_copy_kernel(const CopyParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    int64_t dyn = 0;
    for (int d = 0; d < p.dyn_rank; ++d) {
        int64_t s = p.starts[d];
        s = s < 0 ? 0 : (s > p.dyn_limit[d] ? p.dyn_limit[d] : s);
        dyn += s * p.dyn_str[d];
    }
    int64_t rem = i, io = p.i_off, oo = p.o_off;
    for (int d = p.rank - 1; d >= 0; --d) {
        int64_t c = rem % p.dims[d];
        rem /= p.dims[d];
        io += c * p.i_str[d];
        oo += c * p.o_str[d];
    }
    if (p.dyn_on_out) oo += dyn; else io += dyn;
    static_cast<T*>(p.out)[oo] = static_cast<const T*>(p.in)[io];
}

enum { U_NEG, U_ABS, U_EXP, U_LOG, U_TANH, U_ERF, U_RSQRT, U_RECIP };
enum { B_ADD, B_SUB, B_MUL, B_DIV, B_MAX, B_MIN };
enum { C_LT, C_LE, C_EQ, C_GE, C_GT, C_NE };

struct EwParams { const void* a; const void* b; const void* c; void* out; int64_t n; int op; int is_int; };

__global__ void unary_kernel(const EwParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    if (p.is_int) {
        int x = static_cast<const int*>(p.a)[i];
        static_cast<int*>(p.out)[i] = p.op == U_NEG ? -x : (x < 0 ? -x : x);
        return;
    }
    float x = static_cast<const float*>(p.a)[i], y;
    switch (p.op) {
        case U_NEG: y = -x; break;
        case U_ABS: y = fabsf(x); break;
        case U_EXP: y = expf(x); break;
        case U_LOG: y = logf(x); break;
        case U_TANH: y = tanhf(x); break;
        case U_ERF: y = erff(x); break;
        case U_RSQRT: y = 1.0f / sqrtf(x); break;
        default: y = 1.0f / x; break;
    }
    static_cast<float*>(p.out)[i] = y;
}

__global__ void binary_kernel(const EwParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    if (p.is_int) {
        int a = static_cast<const int*>(p.a)[i], b = static_cast<const int*>(p.b)[i], y;
        switch (p.op) {
            case B_ADD: y = a + b; break;
            case B_SUB: y = a - b; break;
            case B_MUL: y = a * b; break;
            case B_DIV: y = b == 0 ? 0 : a / b; break;
            case B_MAX: y = a > b ? a : b; break;
            default: y = a < b ? a : b; break;
        }
        static_cast<int*>(p.out)[i] = y;
        return;
    }
    float a = static_cast<const float*>(p.a)[i], b = static_cast<const float*>(p.b)[i], y;
    switch (p.op) {
        case B_ADD: y = a + b; break;
        case B_SUB: y = a - b; break;
        case B_MUL: y = a * b; break;
        case B_DIV: y = a / b; break;
        case B_MAX: y = fmaxf(a, b); break;
        default: y = fminf(a, b); break;
    }
    static_cast<float*>(p.out)[i] = y;
}

__global__ void compare_kernel(const EwParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    bool r;
    if (p.is_int) {
        int a = static_cast<const int*>(p.a)[i], b = static_cast<const int*>(p.b)[i];
        r = p.op == C_LT ? a < b : p.op == C_LE ? a <= b : p.op == C_EQ ? a == b : p.op == C_GE ? a >= b : p.op == C_GT ? a > b : a != b;
    } else {
        float a = static_cast<const float*>(p.a)[i], b = static_cast<const float*>(p.b)[i];
        r = p.op == C_LT ? a < b : p.op == C_LE ? a <= b : p.op == C_EQ ? a == b : p.op == C_GE ? a >= b : p.op == C_GT ? a > b : a != b;
    }
    static_cast<uint8_t*>(p.out)[i] = r ? 1 : 0;
}

__global__ void select_kernel(const EwParams p) {  // a: pred (u8), b / c: 4-byte values
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    static_cast<uint32_t*>(p.out)[i] = static_cast<const uint8_t*>(p.a)[i] ? static_cast<const uint32_t*>(p.b)[i]
                                                                           : static_cast<const uint32_t*>(p.c)[i];
}

// op: 0 f32->si32 (truncate, saturate, NaN -> 0), 1 si32->f32, 2 i1->f32, 3 i1->si32, 4 f32->i1, 5 si32->i1,
//     6 f32->bf16, 7 bf16->f32, 8 f32->f16, 9 f16->f32 (round to nearest even)
__global__ void cast_kernel(const EwParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n) return;
    switch (p.op) {
        case 0: {
            float x = static_cast<const float*>(p.a)[i];
            int y = isnan(x) ? 0 : (x >= 2147483648.f ? 2147483647 : (x <= -2147483648.f ? (-2147483647 - 1) : (int)truncf(x)));
            static_cast<int*>(p.out)[i] = y;
            break;
        }
        case 1: static_cast<float*>(p.out)[i] = (float)static_cast<const int*>(p.a)[i]; break;
        case 2: static_cast<float*>(p.out)[i] = static_cast<const uint8_t*>(p.a)[i] ? 1.f : 0.f; break;
        case 3: static_cast<int*>(p.out)[i] = static_cast<const uint8_t*>(p.a)[i] ? 1 : 0; break;
        case 4: static_cast<uint8_t*>(p.out)[i] = static_cast<const float*>(p.a)[i] != 0.f; break;
        case 6: static_cast<__nv_bfloat16*>(p.out)[i] = __float2bfloat16_rn(static_cast<const float*>(p.a)[i]); break;
        case 7: static_cast<float*>(p.out)[i] = __bfloat162float(static_cast<const __nv_bfloat16*>(p.a)[i]); break;
        case 8: static_cast<__half*>(p.out)[i] = __float2half_rn(static_cast<const float*>(p.a)[i]); break;
        case 9: static_cast<float*>(p.out)[i] = __half2float(static_cast<const __half*>(p.a)[i]); break;
        default: static_cast<uint8_t*>(p.out)[i] = static_cast<const int*>(p.a)[i] != 0; break;
    }
}

struct ReduceParams { const void* in; void* out; int64_t outer, axis, inner; int kind; int is_int; };
// One warp per (outer, inner) pair; lanes stride over the reduced axis.
__global__ void reduce_kernel(const ReduceParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t w = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= p.outer * p.inner) return;
    const int64_t o = w / p.inner, in = w % p.inner;
    if (p.is_int) {
        const int* x = static_cast<const int*>(p.in) + o * p.axis * p.inner + in;
        int acc = p.kind == 0 ? 0 : (p.kind == 1 ? (-2147483647 - 1) : 2147483647);
        for (int64_t k = lane; k < p.axis; k += 32) {
            int v = x[k * p.inner];
            acc = p.kind == 0 ? acc + v : (p.kind == 1 ? max(acc, v) : min(acc, v));
        }
        for (int s = 16; s > 0; s >>= 1) {
            int v = __shfl_xor_sync(0xffffffffu, acc, s);
            acc = p.kind == 0 ? acc + v : (p.kind == 1 ? max(acc, v) : min(acc, v));
        }
        if (lane == 0) static_cast<int*>(p.out)[w] = acc;
        return;
    }
    const float* x = static_cast<const float*>(p.in) + o * p.axis * p.inner + in;
    float acc = p.kind == 0 ? 0.f : (p.kind == 1 ? -INFINITY : INFINITY);
    for (int64_t k = lane; k < p.axis; k += 32) {
        float v = x[k * p.inner];
        acc = p.kind == 0 ? acc + v : (p.kind == 1 ? fmaxf(acc, v) : fminf(acc, v));
    }
    for (int s = 16; s > 0; s >>= 1) {
        float v = __shfl_xor_sync(0xffffffffu, acc, s);
        acc = p.kind == 0 ? acc + v : (p.kind == 1 ? fmaxf(acc, v) : fminf(acc, v));
    }
    if (lane == 0) static_cast<float*>(p.out)[w] = acc;
}

// out[b][m][n] = sum_k A[b, m, k] * B[b, k, n] with arbitrary strides (f32); one thread per output.
struct DotParams {
    const float* a; const float* b; float* out;
    int64_t nb, m, k, n;
    int64_t a_sb, a_sm, a_sk, b_sb, b_sk, b_sn;
};
__global__ void dot_kernel(const DotParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.nb * p.m * p.n) return;
    const int64_t n = i % p.n, m = (i / p.n) % p.m, b = i / (p.n * p.m);
    const float* a = p.a + b * p.a_sb + m * p.a_sm;
    const float* bb = p.b + b * p.b_sb + n * p.b_sn;
    float acc = 0.f;
    for (int64_t k = 0; k < p.k; ++k) acc = fmaf(a[k * p.a_sk], bb[k * p.b_sk], acc);
    p.out[i] = acc;
}

struct IotaParams { int* out; int64_t n, inner, dim; };
__global__ void iota_kernel(const IotaParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < p.n) p.out[i] = (int)((i / p.inner) % p.dim);
}

struct TakeParams { const uint32_t* w; const int* idx; uint32_t* out; int64_t n_idx, row, vocab; int* status; };
__global__ void take_kernel(const TakeParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n_idx * p.row) return;
    const int64_t r = i / p.row, c = i % p.row;
    const int id = p.idx[r];
    if (id < 0 || id >= p.vocab) { if (c == 0) atomicExch(p.status, 2); p.out[i] = 0; return; }
    p.out[i] = p.w[(int64_t)id * p.row + c];
}

struct GatherParams { const uint32_t* in; const int* idx; uint32_t* out; int64_t outer, axis_in, axis_out, inner; int* status; };
__global__ void gather_kernel(const GatherParams p) {  // take_along_axis
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.outer * p.axis_out * p.inner) return;
    const int64_t in = i % p.inner, o = i / (p.inner * p.axis_out);
    const int id = p.idx[i];
    if (id < 0 || id >= p.axis_in) { atomicExch(p.status, 2); p.out[i] = 0; return; }
    p.out[i] = p.in[(o * p.axis_in + id) * p.inner + in];
}

// ReduceWindow over a rank-4 f32 tensor (crates/gpt-rs-backend-ref-cpu/src/cpu.rs:1944-2108): one thread per output
// element walks its window; a window position counts when it lands on a base-dilated input element inside the tensor.
struct ReduceWindowParams {
    const float* in; float* out;
    int64_t n_out;
    int in_dims[4], out_dims[4], window[4], stride[4], pad_lo[4], base_dil[4], win_dil[4];
    int kind;  // 0 sum, 1 max, 2 min
};
__global__ void reduce_window_kernel(const ReduceWindowParams p) {
    pdl_launch_dependents();  // dependents still wait for this whole grid before reading its results
    pdl_wait();
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= p.n_out) return;
    int o[4];
    int64_t r = i;
#pragma unroll
    for (int d = 3; d >= 0; --d) { o[d] = (int)(r % p.out_dims[d]); r /= p.out_dims[d]; }
    int start[4];
#pragma unroll
    for (int d = 0; d < 4; ++d) start[d] = o[d] * p.stride[d] - p.pad_lo[d];
    float acc = p.kind == 0 ? 0.f : (p.kind == 1 ? -INFINITY : INFINITY);
    for (int w0 = 0; w0 < p.window[0]; ++w0) {
        const int p0 = start[0] + w0 * p.win_dil[0];
        if (p0 < 0 || p0 % p.base_dil[0] != 0 || p0 / p.base_dil[0] >= p.in_dims[0]) continue;
        for (int w1 = 0; w1 < p.window[1]; ++w1) {
            const int p1 = start[1] + w1 * p.win_dil[1];
            if (p1 < 0 || p1 % p.base_dil[1] != 0 || p1 / p.base_dil[1] >= p.in_dims[1]) continue;
            for (int w2 = 0; w2 < p.window[2]; ++w2) {
                const int p2 = start[2] + w2 * p.win_dil[2];
                if (p2 < 0 || p2 % p.base_dil[2] != 0 || p2 / p.base_dil[2] >= p.in_dims[2]) continue;
                for (int w3 = 0; w3 < p.window[3]; ++w3) {
                    const int p3 = start[3] + w3 * p.win_dil[3];
                    if (p3 < 0 || p3 % p.base_dil[3] != 0 || p3 / p.base_dil[3] >= p.in_dims[3]) continue;
                    const int64_t lin = (((int64_t)(p0 / p.base_dil[0]) * p.in_dims[1] + p1 / p.base_dil[1]) * p.in_dims[2] +
                                         p2 / p.base_dil[2]) * p.in_dims[3] + p3 / p.base_dil[3];
                    const float v = p.in[lin];
                    acc = p.kind == 0 ? acc + v : (p.kind == 1 ? fmaxf(acc, v) : fminf(acc, v));
                }
            }
        }
    }
    p.out[i] = acc;
}

template <typename P>
int launch_flat(void (*k)(P), int64_t n, const P& p, cudaStream_t st) {
    if (n <= 0) return GPTRS_OK;
    // through the common launcher: under a recorded plan the launch carries the programmatic-dependent-launch attribute
    return launch_kernel(k, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, 1, p);
}

std::vector<int64_t> row_major_strides(const std::vector<int64_t>& dims) {
    std::vector<int64_t> s(dims.size(), 1);
    for (int i = (int)dims.size() - 2; i >= 0; --i) s[i] = s[i + 1] * dims[i + 1];
    return s;
}

// ---- the plan --------------------------------------------------------------------------------------
struct Plan {
    Function fn;
    std::unordered_map<uint32_t, int> def;       // value id -> instruction index
    std::unordered_map<uint32_t, int> uses;      // value id -> use count (operands + results)
    int fused = 0;
    // Buffer plan (the counterpart of the reference's liveness-based bufferisation,
    // crates/gpt-rs/src/backend/conversion/bufferize.rs): every temporary of the function gets a fixed offset in ONE
    // arena that is allocated when the plan first runs; two values share bytes when their lifetimes do not overlap.
    // Values that leave the function (results, and what they are views of) are allocated per call.
    std::vector<int64_t> arena_offset;           // per instruction: offset of its value, -1 = allocated per call / a view
    int64_t arena_bytes = 0;
    Tensor* arena = nullptr;                     // retained; one per plan (and so per device)
    int device = 0;
    std::mutex run_mu;                           // the arena serves one execution at a time
    // CUDA graphs of the whole execution. A graph bakes in every pointer, so it is valid for one set of input buffers and
    // one set of result buffers: a replay first asks the pool for the results in the order the recorded run took them and
    // launches the graph only if the pool hands back the very same blocks (in a decode loop the caches ping-pong between
    // two sets of blocks, so two graphs serve every step); otherwise the call runs kernel by kernel as before.
    struct RunGraph {
        std::vector<const void*> in_ptrs;        // data pointers of the inputs
        std::vector<TSpec> allocs;               // the pool allocations of the run, in order
        std::vector<void*> alloc_ptrs;           // ... and the blocks they received
        std::vector<int> result_of;              // result i = allocation result_of[i]
        cudaGraphExec_t exec = nullptr;
        int64_t launches = 0;
    };
    std::vector<RunGraph> graphs;
    // The legacy default stream cannot be captured: graphs are recorded and launched on a stream of the plan's own,
    // ordered after and before the caller's stream with two events.
    cudaStream_t side_stream = nullptr;
    cudaEvent_t ev_in = nullptr, ev_out = nullptr;
    int runs = 0, graph_failures = 0;
    bool graph_ok = true;                        // false once an execution turned out not to fit the scheme
    ~Plan() {
        for (auto& g : graphs) if (g.exec) cudaGraphExecDestroy(g.exec);
        if (ev_in) cudaEventDestroy(ev_in);
        if (ev_out) cudaEventDestroy(ev_out);
        if (side_stream) cudaStreamDestroy(side_stream);
        tensor_release(arena);
    }
};

const Inst* def_of(const Plan& pl, const Operand& o) {
    if (o.is_literal) return nullptr;
    auto it = pl.def.find(o.id);
    return it == pl.def.end() ? nullptr : &pl.fn.body[it->second];
}
int uses_of(const Plan& pl, uint32_t id) { auto it = pl.uses.find(id); return it == pl.uses.end() ? 0 : it->second; }
bool is_bin(const Inst* i, const char* k) { return i && !i->dead && i->op == Op::Binary && i->sub == k; }
bool is_un(const Inst* i, const char* k) { return i && !i->dead && i->op == Op::Unary && i->sub == k; }
bool is_red(const Inst* i, const char* k) {
    return i && !i->dead && i->op == Op::Reduce && i->sub == k && i->keepdims && i->a.size() == 1 &&
           !i->operands.empty() && !i->operands[0].is_literal;
}
bool same_val(const Operand& a, const Operand& b) { return !a.is_literal && !b.is_literal && a.id == b.id; }

// BroadcastTo chain ending in a scalar f32 literal: returns true and the value.
bool scalar_literal(const Plan& pl, const Operand& o, float* v) {
    const Operand* cur = &o;
    for (int depth = 0; depth < 4; ++depth) {
        if (cur->is_literal) {
            if (cur->lit.dtype != GPTRS_F32 || cur->lit.numel() != 1 || cur->bytes.size() != 4) return false;
            memcpy(v, cur->bytes.data(), 4);
            return true;
        }
        const Inst* d = def_of(pl, *cur);
        if (!d || d->op != Op::BroadcastTo || d->operands.size() != 1) return false;
        cur = &d->operands[0];
    }
    return false;
}

// BroadcastTo(x.shape) of a rank-1 [D] tensor (gamma / beta): returns the source operand.
const Operand* row_broadcast(const Plan& pl, const Operand& o, int64_t d) {
    const Inst* b = def_of(pl, o);
    if (!b || b->dead || b->op != Op::BroadcastTo || b->operands[0].is_literal) return nullptr;
    auto it = pl.def.find(b->operands[0].id);
    const TSpec* src = nullptr;
    if (it != pl.def.end()) src = &pl.fn.body[it->second].out;
    else
        for (size_t i = 0; i < pl.fn.param_ids.size(); ++i)
            if (pl.fn.param_ids[i] == b->operands[0].id) src = &pl.fn.params[i];
    if (!src || src->dims.size() != 1 || src->dims[0] != d) return nullptr;
    return &b->operands[0];
}

// Matches inv = Rsqrt(Add(Mul(ReduceSum(sq_src . sq_src), c), eps)) broadcast back to x's shape, where the
// squared operand is `sq_of`. Returns eps through *eps.
bool match_inv_scale(const Plan& pl, const Operand& o, const Operand& sq_of, int64_t n, float* eps) {
    const Inst* bc = def_of(pl, o);
    if (!bc || bc->dead || bc->op != Op::BroadcastTo) return false;
    const Inst* rs = def_of(pl, bc->operands[0]);
    if (!is_un(rs, "Rsqrt")) return false;
    const Inst* add = def_of(pl, rs->operands[0]);
    if (!is_bin(add, "Add")) return false;
    for (int sw = 0; sw < 2; ++sw) {
        const Operand& var_o = add->operands[sw];
        const Operand& eps_o = add->operands[1 - sw];
        float e;
        if (!scalar_literal(pl, eps_o, &e)) continue;
        const Inst* mul = def_of(pl, var_o);
        if (!is_bin(mul, "Mul")) continue;
        for (int sw2 = 0; sw2 < 2; ++sw2) {
            float c;
            if (!scalar_literal(pl, mul->operands[1 - sw2], &c)) continue;
            if (fabsf(c * (float)n - 1.f) > 1e-5f) continue;
            const Inst* red = def_of(pl, mul->operands[sw2]);
            if (!is_red(red, "Sum")) continue;
            const Inst* sq = def_of(pl, red->operands[0]);
            if (!is_bin(sq, "Mul") || !same_val(sq->operands[0], sq->operands[1]) || !same_val(sq->operands[0], sq_of)) continue;
            if (red->a[0] != (int64_t)sq->out.dims.size() - 1) continue;
            *eps = e;
            return true;
        }
    }
    return false;
}

void count_uses(Plan& pl) {
    pl.uses.clear();
    pl.def.clear();
    for (size_t i = 0; i < pl.fn.body.size(); ++i) {
        const Inst& in = pl.fn.body[i];
        if (in.dead) continue;
        pl.def[in.id] = (int)i;
        if (in.side_id) pl.def[in.side_id] = (int)i;
        for (auto& o : in.operands)
            if (!o.is_literal) ++pl.uses[o.id];
    }
    for (uint32_t r : pl.fn.result_ids) ++pl.uses[r];
}

// Marks instructions whose values are no longer used as dead (repeat to a fixed point).
void sweep_dead(Plan& pl) {
    for (;;) {
        count_uses(pl);
        bool changed = false;
        for (auto& in : pl.fn.body)
            if (!in.dead && uses_of(pl, in.id) == 0) { in.dead = true; changed = true; }
        if (!changed) return;
    }
}

// ---- decode attention over a dense cache (functional::attention_decode_cache, attention.rs:657-779) -------------
// The captured graph is
//   scores = DotGeneral(q[Hq,1,hd], KG[Hq,cap,hd])   KG = Reshape(BroadcastTo(Reshape(Slice?(k_cache[Hkv,cap,hd]))))
//   z      = scores * (1/sqrt(hd)) + mask             mask = bcast(Select(bcast(DynamicSlice(iota, query_start)) >= iota, 0, -1e9))
//   ctx    = DotGeneral(Softmax(z), VG[Hq,cap,hd])    VG built like KG from v_cache
// It materialises two [Hq, cap, hd] copies of the caches and a [Hq, cap] score row per step. The helpers below
// recognise it so that one kernel can read k_cache / v_cache in place.

const TSpec* spec_of(const Plan& pl, const Operand& o) {
    if (o.is_literal) return nullptr;
    auto it = pl.def.find(o.id);
    if (it != pl.def.end()) return &pl.fn.body[it->second].out;
    for (size_t i = 0; i < pl.fn.param_ids.size(); ++i)
        if (pl.fn.param_ids[i] == o.id) return &pl.fn.params[i];
    return nullptr;
}

// KG / VG -> the [Hkv, cap, hd] cache it repeats per query-head group.
const Operand* grouped_cache_source(const Plan& pl, const Operand& o, int64_t hq, int64_t cap, int64_t hd, int64_t* hkv) {
    const Inst* r2 = def_of(pl, o);
    if (!r2 || r2->dead || r2->op != Op::Reshape || r2->out.dims != std::vector<int64_t>{hq, cap, hd}) return nullptr;
    const Inst* bc = def_of(pl, r2->operands[0]);
    if (!bc || bc->dead || bc->op != Op::BroadcastTo || bc->out.dims.size() != 4) return nullptr;
    const int64_t kv = bc->out.dims[0], grp = bc->out.dims[1];
    if (kv * grp != hq || bc->out.dims[2] != cap || bc->out.dims[3] != hd) return nullptr;
    const Inst* r1 = def_of(pl, bc->operands[0]);
    if (!r1 || r1->dead || r1->op != Op::Reshape || r1->out.dims != std::vector<int64_t>{kv, 1, cap, hd}) return nullptr;
    const Operand* src = &r1->operands[0];
    const Inst* sl = def_of(pl, *src);
    if (sl && !sl->dead && sl->op == Op::Slice) {  // a slice of the whole tensor
        const TSpec* in_spec = spec_of(pl, sl->operands[0]);
        if (!in_spec || in_spec->dims != sl->out.dims) return nullptr;
        for (int64_t st : sl->a) if (st != 0) return nullptr;
        src = &sl->operands[0];
    }
    const TSpec* cs = spec_of(pl, *src);
    if (!cs || cs->dtype != GPTRS_F32 || cs->dims != std::vector<int64_t>{kv, cap, hd}) return nullptr;
    *hkv = kv;
    return src;
}

// The causal mask of one query row; returns the operand holding the query position (si32 [1]).
const Operand* causal_mask_start(const Plan& pl, const Operand& o, int64_t cap) {
    const Operand* cur = &o;
    const Inst* sel = nullptr;
    for (int depth = 0; depth < 4; ++depth) {
        const Inst* d = def_of(pl, *cur);
        if (!d || d->dead) return nullptr;
        if (d->op == Op::BroadcastTo) { cur = &d->operands[0]; continue; }
        if (d->op == Op::Select) sel = d;
        break;
    }
    if (!sel || sel->operands.size() != 3 || sel->out.dims != std::vector<int64_t>{cap}) return nullptr;
    float keep, drop;
    if (!scalar_literal(pl, sel->operands[1], &keep) || !scalar_literal(pl, sel->operands[2], &drop)) return nullptr;
    if (keep != 0.f || drop > -1e8f) return nullptr;
    const Inst* cmp = def_of(pl, sel->operands[0]);
    if (!cmp || cmp->dead || cmp->op != Op::Compare || cmp->sub != "GreaterEqual") return nullptr;
    const Inst* keys = def_of(pl, cmp->operands[1]);
    if (!keys || keys->dead || keys->op != Op::Iota || keys->out.dims != std::vector<int64_t>{cap}) return nullptr;
    const Inst* qb = def_of(pl, cmp->operands[0]);
    if (!qb || qb->dead || qb->op != Op::BroadcastTo) return nullptr;
    const Inst* ds = def_of(pl, qb->operands[0]);
    if (!ds || ds->dead || ds->op != Op::DynamicSlice || ds->operands.size() != 2 || ds->out.dims != std::vector<int64_t>{1}) return nullptr;
    const Inst* src = def_of(pl, ds->operands[0]);
    if (!src || src->dead || src->op != Op::Iota || src->out.dims != std::vector<int64_t>{cap}) return nullptr;
    const TSpec* st = spec_of(pl, ds->operands[1]);
    if (!st || st->dtype != GPTRS_SI32 || st->numel() != 1) return nullptr;
    return &ds->operands[1];
}

bool is_batched_dot(const Inst* d, int64_t contract_rhs) {
    return d && !d->dead && d->op == Op::DotGeneral && d->a == std::vector<int64_t>{0} && d->b == std::vector<int64_t>{0} &&
           d->c == std::vector<int64_t>{2} && d->d == std::vector<int64_t>{contract_rhs};
}

// Anchor: ctx = DotGeneral(p, VG). On success `in` becomes FusedAttentionDecode(q, k_cache, v_cache, query_start).
bool rewrite_attention_decode(Plan& pl, Inst& in) {
    if (!is_batched_dot(&in, 1) || in.out.dims.size() != 3 || in.out.dims[1] != 1) return false;
    const int64_t hq = in.out.dims[0], hd = in.out.dims[2];
    // geometries the dense-cache attention kernel does not take stay on the op-by-op path
    if (hd > 128) return false;
    const Inst* sm = def_of(pl, in.operands[0]);
    if (!sm || sm->dead || sm->op != Op::FusedSoftmax || sm->out.dims.size() != 3 || sm->out.dims[0] != hq || sm->out.dims[1] != 1) return false;
    const int64_t cap = sm->out.dims[2];
    if (cap > 32768) return false;
    int64_t hkv_v = 0, hkv_k = 0;
    const Operand* v_cache = grouped_cache_source(pl, in.operands[1], hq, cap, hd, &hkv_v);
    const Inst* z = def_of(pl, sm->operands[0]);
    if (!v_cache || !is_bin(z, "Add")) return false;
    for (int sw = 0; sw < 2; ++sw) {
        const Operand* start = causal_mask_start(pl, z->operands[1 - sw], cap);
        const Inst* scaled = def_of(pl, z->operands[sw]);
        if (!start || !is_bin(scaled, "Mul")) continue;
        for (int sw2 = 0; sw2 < 2; ++sw2) {
            float scale;
            const Inst* scores = def_of(pl, scaled->operands[sw2]);
            if (!scalar_literal(pl, scaled->operands[1 - sw2], &scale) || !is_batched_dot(scores, 2)) continue;
            if (fabsf(scale * sqrtf((float)hd) - 1.f) > 1e-5f) continue;
            const Operand& q = scores->operands[0];
            const TSpec* qs = spec_of(pl, q);
            const Operand* k_cache = grouped_cache_source(pl, scores->operands[1], hq, cap, hd, &hkv_k);
            if (!qs || qs->dtype != GPTRS_F32 || qs->dims != std::vector<int64_t>{hq, 1, hd} || !k_cache || hkv_k != hkv_v) continue;
            Inst f = in;
            f.op = Op::FusedAttentionDecode;
            f.operands = {q, *k_cache, *v_cache, *start};
            f.a = {hq, hkv_k, hd, cap};
            in = f;
            ++pl.fused;
            return true;
        }
    }
    return false;
}

// Pattern rewrites. Each replaces the anchor instruction by a fused operation; the interior
// instructions die in sweep_dead() when nothing else uses them (so values that escape stay).
void rewrite_pass(Plan& pl, bool rms_pass) {
    count_uses(pl);
    for (auto& in : pl.fn.body) {
        if (in.dead || in.out.dtype != GPTRS_F32 || in.out.dims.empty()) continue;
        if (!rms_pass && in.op == Op::DotGeneral && rewrite_attention_decode(pl, in)) continue;  // its softmax precedes it
        const int64_t d = in.out.dims.back();
        // ---- rms_norm: Mul(Mul(x, bcast(inv)), bcast(gamma)) ------------------------------------
        if (rms_pass && is_bin(&in, "Mul")) {
            bool done = false;
            for (int sw = 0; sw < 2 && !done; ++sw) {
                const Operand* gamma = row_broadcast(pl, in.operands[1 - sw], d);
                const Inst* nrm = def_of(pl, in.operands[sw]);
                if (!gamma || !is_bin(nrm, "Mul")) continue;
                for (int sw2 = 0; sw2 < 2 && !done; ++sw2) {
                    const Operand& x = nrm->operands[sw2];
                    float eps;
                    if (x.is_literal || !match_inv_scale(pl, nrm->operands[1 - sw2], x, d, &eps)) continue;
                    Inst f = in;
                    f.op = Op::FusedRmsNorm; f.f0 = eps;
                    f.operands = {x, *gamma};
                    in = f; ++pl.fused; done = true;
                }
            }
            if (done) continue;
        }
        if (rms_pass) continue;
        // ---- layer_norm: Add(Mul(Mul(centered, bcast(inv)), bcast(gamma)), bcast(beta)) -----------
        if (is_bin(&in, "Add")) {
            bool done = false;
            for (int sw = 0; sw < 2 && !done; ++sw) {
                const Operand* beta = row_broadcast(pl, in.operands[1 - sw], d);
                const Inst* ng = def_of(pl, in.operands[sw]);
                if (!beta || !is_bin(ng, "Mul")) continue;
                for (int sw2 = 0; sw2 < 2 && !done; ++sw2) {
                    const Operand* gamma = row_broadcast(pl, ng->operands[1 - sw2], d);
                    const Inst* nrm = def_of(pl, ng->operands[sw2]);
                    if (!gamma || !is_bin(nrm, "Mul")) continue;
                    for (int sw3 = 0; sw3 < 2 && !done; ++sw3) {
                        const Operand& cen_o = nrm->operands[sw3];
                        const Inst* cen = def_of(pl, cen_o);
                        float eps;
                        if (!is_bin(cen, "Sub") || !match_inv_scale(pl, nrm->operands[1 - sw3], cen_o, d, &eps)) continue;
                        // centered = Sub(x, bcast(Mul(ReduceSum(x), 1/N)))
                        const Operand& x = cen->operands[0];
                        const Inst* mb = def_of(pl, cen->operands[1]);
                        if (x.is_literal || !mb || mb->op != Op::BroadcastTo) continue;
                        const Inst* mean = def_of(pl, mb->operands[0]);
                        if (!is_bin(mean, "Mul")) continue;
                        bool ok = false;
                        for (int sw4 = 0; sw4 < 2; ++sw4) {
                            float c;
                            const Inst* red = def_of(pl, mean->operands[sw4]);
                            if (scalar_literal(pl, mean->operands[1 - sw4], &c) && fabsf(c * (float)d - 1.f) <= 1e-5f &&
                                is_red(red, "Sum") && same_val(red->operands[0], x) &&
                                red->a[0] == (int64_t)in.out.dims.size() - 1)
                                ok = true;
                        }
                        if (!ok) continue;
                        Inst f = in;
                        f.op = Op::FusedLayerNorm; f.f0 = eps;
                        f.operands = {x, *gamma, *beta};
                        in = f; ++pl.fused; done = true;
                    }
                }
            }
            if (done) continue;
            // ---- matmul + add_bias: Add(DotGeneral[2-D](x, w), bcast(bias)) ---------------------
            for (int sw = 0; sw < 2 && !done; ++sw) {
                const Operand* bias = row_broadcast(pl, in.operands[1 - sw], d);
                const Inst* dot = def_of(pl, in.operands[sw]);
                if (!bias || !dot || dot->dead || dot->op != Op::DotGeneral || in.out.dims.size() != 2) continue;
                if (!dot->a.empty() || dot->c != std::vector<int64_t>{1} || dot->d != std::vector<int64_t>{0}) continue;
                if (uses_of(pl, dot->id) != 1) continue;
                Inst f = in;
                f.op = Op::FusedMatmulBias;
                f.operands = {dot->operands[0], dot->operands[1], *bias};
                in = f; ++pl.fused; done = true;
            }
            if (done) continue;
        }
        // ---- gelu (erf form, activation.rs:96-113): Mul(Mul(x, 0.5), Add(Erf(Div(x, sqrt 2)), 1)), operands either way ----
        if (is_bin(&in, "Mul") && in.out.dtype == GPTRS_F32) {
            bool done = false;
            for (int sw = 0; sw < 2 && !done; ++sw) {
                const Inst* half = def_of(pl, in.operands[sw]);
                const Inst* onep = def_of(pl, in.operands[1 - sw]);
                if (!is_bin(half, "Mul") || !is_bin(onep, "Add")) continue;
                for (int sw2 = 0; sw2 < 2 && !done; ++sw2) {
                    float c05, c1, c2;
                    if (half->operands[sw2].is_literal || !scalar_literal(pl, half->operands[1 - sw2], &c05) || c05 != 0.5f) continue;
                    const Operand& x = half->operands[sw2];
                    for (int sw3 = 0; sw3 < 2 && !done; ++sw3) {
                        const Inst* erf = def_of(pl, onep->operands[sw3]);
                        if (!is_un(erf, "Erf") || !scalar_literal(pl, onep->operands[1 - sw3], &c1) || c1 != 1.f) continue;
                        const Inst* div = def_of(pl, erf->operands[0]);
                        if (!is_bin(div, "Div") || !same_val(div->operands[0], x) || !scalar_literal(pl, div->operands[1], &c2) ||
                            fabsf(c2 - 1.4142135f) > 1e-6f)
                            continue;
                        Inst f = in;
                        f.op = Op::FusedGelu;
                        f.operands = {x};
                        in = f; ++pl.fused; done = true;
                    }
                }
            }
            if (done) continue;
        }
        // ---- softmax over the last axis: Div(e, bcast(ReduceSum(e))), e = Exp(Sub(z, bcast(ReduceMax(z))))
        if (is_bin(&in, "Div")) {
            const Inst* e = def_of(pl, in.operands[0]);
            const Inst* sb = def_of(pl, in.operands[1]);
            if (!is_un(e, "Exp") || !sb || sb->op != Op::BroadcastTo) continue;
            const Inst* rs = def_of(pl, sb->operands[0]);
            if (!is_red(rs, "Sum") || !same_val(rs->operands[0], in.operands[0]) || rs->a[0] != (int64_t)in.out.dims.size() - 1) continue;
            const Inst* sub = def_of(pl, e->operands[0]);
            if (!is_bin(sub, "Sub")) continue;
            const Inst* mb = def_of(pl, sub->operands[1]);
            if (!mb || mb->op != Op::BroadcastTo) continue;
            const Inst* rm = def_of(pl, mb->operands[0]);
            if (!is_red(rm, "Max") || !same_val(rm->operands[0], sub->operands[0]) || rm->a[0] != (int64_t)in.out.dims.size() - 1) continue;
            Inst f = in;
            f.op = Op::FusedSoftmax;
            f.operands = {sub->operands[0]};
            in = f; ++pl.fused;
        }
    }
    sweep_dead(pl);
    // gelu of a matmul + bias that nothing else reads: the activation moves into the matmul's epilogue
    for (auto& in : pl.fn.body) {
        if (in.dead || in.op != Op::FusedGelu) continue;
        const Inst* mm = def_of(pl, in.operands[0]);
        if (!mm || mm->dead || mm->op != Op::FusedMatmulBias || mm->axis == 1 || uses_of(pl, mm->id) != 1) continue;
        Inst f = in;
        f.op = Op::FusedMatmulBias;
        f.axis = 1;
        f.operands = mm->operands;
        in = f;
    }
    sweep_dead(pl);
}

// dequant + dot_general: DotGeneral(x[M,K], W) with W = Dequantize(q, scales)[N,K] contracted over K, directly or
// through Transpose([1,0]) (the Linear layout [K,N]) -> FusedQuantMatmul(x, q, scales): the f32 weight is never built.
void rewrite_quant_dots(Plan& pl) {
    count_uses(pl);
    for (auto& in : pl.fn.body) {
        if (in.dead || in.op != Op::DotGeneral || in.out.dtype != GPTRS_F32 || in.out.dims.size() != 2) continue;
        if (!in.a.empty() || in.c != std::vector<int64_t>{1} || in.d.size() != 1) continue;
        const TSpec* xs = spec_of(pl, in.operands[0]);
        if (!xs || xs->dtype != GPTRS_F32 || xs->dims.size() != 2) continue;
        const Inst* w = def_of(pl, in.operands[1]);
        int64_t contract = in.d[0];
        if (w && !w->dead && w->op == Op::Transpose && w->a == std::vector<int64_t>{1, 0}) { w = def_of(pl, w->operands[0]); contract = 1 - contract; }
        if (!w || w->dead || w->op != Op::Dequantize || contract != 1 || w->operands.size() != 2) continue;
        const int64_t n = w->out.dims[0], k = w->out.dims[1];
        if (k % 128 != 0 || n % 16 != 0 || xs->dims[1] != k) continue;
        Inst f = in;
        f.op = Op::FusedQuantMatmul;
        f.sub = spec_of(pl, w->operands[0])->dtype == GPTRS_SI8 ? "w8" : "w4";
        f.operands = {in.operands[0], w->operands[0], w->operands[1]};
        in = f;
        ++pl.fused;
    }
    sweep_dead(pl);
}

// norm + residual: FusedRmsNorm / FusedLayerNorm whose input is Add(residual, update) -> one kernel that adds and
// normalises. When the sum has other readers (it is the new residual stream) the kernel writes it as a second result,
// provided none of those readers comes before the norm in the instruction order.
void rewrite_add_norms(Plan& pl, bool allow_second_result) {
    count_uses(pl);
    for (size_t i = 0; i < pl.fn.body.size(); ++i) {
        Inst& in = pl.fn.body[i];
        if (in.dead || (in.op != Op::FusedRmsNorm && in.op != Op::FusedLayerNorm) || in.operands[0].is_literal) continue;
        auto it = pl.def.find(in.operands[0].id);
        if (it == pl.def.end()) continue;
        Inst& add = pl.fn.body[it->second];
        if (!is_bin(&add, "Add") || add.out.dtype != GPTRS_F32 || add.operands[0].is_literal || add.operands[1].is_literal) continue;
        bool early_reader = false, is_result = false;
        for (size_t j = 0; j < i; ++j)
            for (const Operand& o : pl.fn.body[j].operands)
                if (!pl.fn.body[j].dead && !o.is_literal && o.id == add.id) early_reader = true;
        for (uint32_t r : pl.fn.result_ids) is_result = is_result || r == add.id;
        if (early_reader) continue;
        const bool shared = uses_of(pl, add.id) > 1 || is_result;
        if (shared && !allow_second_result) continue;   // the text form of a CustomCall has one result
        Inst f = in;
        f.op = in.op == Op::FusedRmsNorm ? Op::FusedAddRmsNorm : Op::FusedAddLayerNorm;
        f.operands = {add.operands[0], add.operands[1]};
        for (size_t k = 1; k < in.operands.size(); ++k) f.operands.push_back(in.operands[k]);
        if (shared) { f.side_id = add.id; f.side_out = add.out; }
        add.dead = true;
        in = f;
        ++pl.fused;
        count_uses(pl);
    }
    sweep_dead(pl);
}

// layer_norm / softmax / matmul+bias first: a layer_norm contains an rms_norm-shaped subgraph.
void rewrite(Plan& pl, bool in_process = true) {
    rewrite_pass(pl, false);
    rewrite_pass(pl, true);
    rewrite_quant_dots(pl);
    rewrite_add_norms(pl, in_process);
}

// True for operations whose result is (or may be) the storage of an operand: their source must live as long as they do.
bool may_alias_operand(const Inst& in) {
    return in.op == Op::Reshape || in.op == Op::Constant || in.op == Op::StopGradient || in.op == Op::Cast;
}

// Assigns arena offsets (see Plan). Lifetimes are instruction indices; a value that an aliasing operation forwards
// lives as long as the alias. First-fit over the blocks free at the defining instruction.
void plan_buffers(Plan& pl) {
    const auto& body = pl.fn.body;
    const int n = (int)body.size();
    pl.arena_offset.assign(n, -1);
    std::vector<int> last(n, -1);          // last instruction index that reads the value of instruction i
    std::vector<char> escapes(n, 0);
    auto idx_of = [&](uint32_t id) { auto it = pl.def.find(id); return it == pl.def.end() ? -1 : it->second; };
    for (uint32_t r : pl.fn.result_ids) { int i = idx_of(r); if (i >= 0) escapes[i] = 1; }
    for (int i = n - 1; i >= 0; --i) {
        const Inst& in = body[i];
        if (in.dead) continue;
        for (const Operand& o : in.operands) {
            if (o.is_literal) continue;
            const int src = idx_of(o.id);
            if (src < 0) continue;
            last[src] = std::max(last[src], i);
            if (may_alias_operand(in)) {   // the alias keeps its source alive and passes an escape on
                last[src] = std::max(last[src], last[i]);
                if (escapes[i]) escapes[src] = 1;
            }
        }
    }
    struct Block { int64_t off, bytes; int free_at; };
    std::vector<Block> blocks;
    int64_t top = 0;
    for (int i = 0; i < n; ++i) {
        const Inst& in = body[i];
        if (in.dead || escapes[i] || may_alias_operand(in)) continue;
        int64_t bytes = (((int64_t)in.out.numel() * (int64_t)dtype_size(in.out.dtype)) + 255) & ~(int64_t)255;
        // a second result (the sum of a fused residual-add + norm) lives right behind the first, for the same lifetime
        // (value ids of both map to this instruction, so `last` already covers the readers of either)
        if (in.side_id) bytes += (((int64_t)in.side_out.numel() * (int64_t)dtype_size(in.side_out.dtype)) + 255) & ~(int64_t)255;
        // the bf16 copy of the activations that a quantised matmul reads lives right behind its result
        if (in.op == Op::FusedQuantMatmul && !in.operands.empty()) {
            const TSpec* xs = spec_of(pl, in.operands[0]);
            if (xs) bytes += ((xs->numel() * 2) + 255) & ~(int64_t)255;
        }
        if (bytes == 0) continue;
        const int free_at = last[i] < 0 ? i : last[i];
        int best = -1;
        for (int b = 0; b < (int)blocks.size(); ++b)
            if (blocks[b].free_at < i && blocks[b].bytes >= bytes && (best < 0 || blocks[b].bytes < blocks[best].bytes)) best = b;
        if (best >= 0) {
            pl.arena_offset[i] = blocks[best].off;
            blocks[best].free_at = free_at;
        } else {
            pl.arena_offset[i] = top;
            blocks.push_back({top, bytes, free_at});
            top += bytes;
        }
    }
    pl.arena_bytes = top;
}

// Literal operands are uploaded once per plan.
int upload_literals(Plan& pl) {
    for (auto& in : pl.fn.body) {
        if (in.dead) continue;
        for (auto& o : in.operands) {
            if (!o.is_literal || o.device) continue;
            Tensor* t = nullptr;
            int rc = tensor_alloc(o.lit.dtype, (int)o.lit.dims.size(), o.lit.dims.data(), false, &t);
            if (rc) return rc;
            if (o.bytes.size() != t->bytes) { tensor_release(t); return fail(GPTRS_SPEC_VIOLATION, "literal byte length mismatch"); }
            if (t->bytes && cudaMemcpy(t->data, o.bytes.data(), t->bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
                tensor_release(t);
                return fail(GPTRS_EXECUTION, "literal upload failed");
            }
            o.device = t;
        }
    }
    return GPTRS_OK;
}

uint64_t fnv1a(const char* s, size_t n) {
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < n; ++i) { h ^= (unsigned char)s[i]; h *= 1099511628211ull; }
    return h;
}

std::mutex g_plan_mu;
std::unordered_map<uint64_t, std::shared_ptr<Plan>> g_plans;
int64_t g_plan_hits = 0, g_plan_builds = 0, g_last_launches = 0, g_last_fused = 0;
int g_fusion_enabled = 1;
int g_arena_enabled = 1;   // GPTRS_PTIR_ARENA=0 allocates every temporary by itself (for comparison)

int* status_word() {
    static int* d = nullptr;
    if (!d) { if (cudaMalloc(&d, 4) != cudaSuccess) return nullptr; cudaMemset(d, 0, 4); }
    return d;
}

// ---- execution -------------------------------------------------------------------------------------
struct Exec {
    cudaStream_t st;
    std::unordered_map<uint32_t, Tensor*> env;  // retained
    int64_t launches = 0;
    Tensor* arena = nullptr;      // the plan's arena (not retained here: the plan outlives the execution)
    int64_t arena_off = -1;       // offset of the value of the instruction being executed, -1 = allocate
    Tensor* side = nullptr;       // second result of the instruction being executed (retained), if it has one
    ~Exec() { for (auto& kv : env) tensor_release(kv.second); }

    int value(const Operand& o, Tensor** out) {  // returns a retained tensor
        if (o.is_literal) {
            Tensor* t = static_cast<Tensor*>(o.device);
            if (!t) return fail(GPTRS_EXECUTION, "literal was not uploaded");
            tensor_retain(t);
            *out = t;
            return GPTRS_OK;
        }
        auto it = env.find(o.id);
        if (it == env.end()) return fail(GPTRS_SPEC_VIOLATION, "use of undefined value %" + std::to_string(o.id));
        tensor_retain(it->second);
        *out = it->second;
        return GPTRS_OK;
    }
};

int copy_generic(Exec& ex, const Tensor* in, Tensor* out, const std::vector<int64_t>& dims, const std::vector<int64_t>& i_str,
                 const std::vector<int64_t>& o_str, int64_t i_off, int64_t o_off, const int* starts = nullptr,
                 const std::vector<int64_t>& dyn_limit = {}, const std::vector<int64_t>& dyn_str = {}, bool dyn_on_out = false) {
    if (dims.size() > (size_t)kMaxRank) return fail(GPTRS_UNIMPLEMENTED, "rank above 8");
    CopyParams p = {};
    p.in = in->data; p.out = out->data; p.rank = (int)dims.size();
    p.n = 1;
    for (size_t d = 0; d < dims.size(); ++d) { p.dims[d] = dims[d]; p.i_str[d] = i_str[d]; p.o_str[d] = o_str[d]; p.n *= dims[d]; }
    p.i_off = i_off; p.o_off = o_off;
    p.starts = starts; p.dyn_rank = (int)dyn_limit.size(); p.dyn_on_out = dyn_on_out;
    for (size_t d = 0; d < dyn_limit.size(); ++d) { p.dyn_limit[d] = dyn_limit[d]; p.dyn_str[d] = dyn_str[d]; }
    ++ex.launches;
    const size_t es = dtype_size(in->dtype);
    return es == 4 ? launch_flat(strided_copy_kernel<uint32_t>, p.n, p, ex.st)
           : es == 2 ? launch_flat(strided_copy_kernel<uint16_t>, p.n, p, ex.st)
                     : launch_flat(strided_copy_kernel<uint8_t>, p.n, p, ex.st);
}

int exec_inst(Exec& ex, const Inst& in, std::vector<Tensor*>& ops, Tensor** result) {
    auto unimpl = [&](const std::string& why) { return fail(GPTRS_UNIMPLEMENTED, in.name + " is not implemented: " + why); };
    auto spec = [&](const std::string& why) { return fail(GPTRS_SPEC_VIOLATION, in.name + " (%" + std::to_string(in.id) + "): " + why); };
    Tensor* out = nullptr;
    auto alloc_out = [&]() {
        if (ex.arena && ex.arena_off >= 0) {   // a temporary with a planned place in the arena
            out = new Tensor();
            out->dtype = in.out.dtype; out->dims = in.out.dims;
            out->bytes = (size_t)in.out.numel() * dtype_size(in.out.dtype);
            out->data = static_cast<unsigned char*>(ex.arena->data) + ex.arena_off;
            out->owns = false; out->base = ex.arena; out->device = ex.arena->device;
            tensor_retain(ex.arena);
            return (int)GPTRS_OK;
        }
        return tensor_alloc(in.out.dtype, (int)in.out.dims.size(), in.out.dims.data(), false, &out);
    };
    const int64_t n_out = in.out.numel();
    int rc = GPTRS_OK;
    switch (in.op) {
        case Op::Constant:
        case Op::StopGradient:
            tensor_retain(ops[0]);
            *result = ops[0];
            return GPTRS_OK;
        case Op::Reshape: {
            if (ops[0]->numel() != n_out) return spec("element count changes");
            Tensor* t = new Tensor();
            t->dtype = ops[0]->dtype; t->dims = in.out.dims; t->data = ops[0]->data; t->bytes = ops[0]->bytes;
            t->owns = false; t->base = ops[0];
            tensor_retain(ops[0]);
            *result = t;
            return GPTRS_OK;
        }
        case Op::Unary: case Op::Binary: case Op::Compare: case Op::Select: case Op::Cast: {
            if ((rc = alloc_out())) return rc;
            EwParams p = {};
            p.n = n_out; p.out = out->data; p.a = ops[0]->data;
            ++ex.launches;
            if (in.op == Op::Unary) {
                static const char* names[] = {"Neg", "Abs", "Exp", "Log", "Tanh", "Erf", "Rsqrt", "Reciprocal"};
                p.op = -1;
                for (int i = 0; i < 8; ++i) if (in.sub == names[i]) p.op = i;
                p.is_int = ops[0]->dtype == GPTRS_SI32;
                if (p.op < 0 || (p.is_int && p.op > U_ABS) || ops[0]->dtype == GPTRS_I1) { tensor_release(out); return unimpl("unary " + in.sub + " on this dtype"); }
                rc = launch_flat(unary_kernel, p.n, p, ex.st);
            } else if (in.op == Op::Binary || in.op == Op::Compare) {
                if (ops[0]->dims != ops[1]->dims || ops[0]->dtype != ops[1]->dtype) { tensor_release(out); return spec("operand shapes or dtypes differ"); }
                p.b = ops[1]->data; p.is_int = ops[0]->dtype == GPTRS_SI32;
                if (ops[0]->dtype == GPTRS_I1) { tensor_release(out); return unimpl("i1 operands"); }
                if (in.op == Op::Binary) {
                    static const char* names[] = {"Add", "Sub", "Mul", "Div", "Maximum", "Minimum"};
                    p.op = -1;
                    for (int i = 0; i < 6; ++i) if (in.sub == names[i]) p.op = i;
                    if (p.op < 0) { tensor_release(out); return unimpl("binary " + in.sub); }
                    rc = launch_flat(binary_kernel, p.n, p, ex.st);
                } else {
                    static const char* names[] = {"Less", "LessEqual", "Equal", "GreaterEqual", "Greater", "NotEqual"};
                    p.op = -1;
                    for (int i = 0; i < 6; ++i) if (in.sub == names[i]) p.op = i;
                    if (p.op < 0) { tensor_release(out); return unimpl("compare " + in.sub); }
                    rc = launch_flat(compare_kernel, p.n, p, ex.st);
                }
            } else if (in.op == Op::Select) {
                if (ops[0]->dtype != GPTRS_I1 || dtype_size(ops[1]->dtype) != 4 || ops[1]->dims != ops[2]->dims || ops[0]->dims != ops[1]->dims) {
                    tensor_release(out); return spec("select needs an i1 predicate and equal 4-byte branches");
                }
                p.b = ops[1]->data; p.c = ops[2]->data;
                rc = launch_flat(select_kernel, p.n, p, ex.st);
            } else {
                const int from = ops[0]->dtype, to = in.out.dtype;
                if (from == to) { tensor_release(out); tensor_retain(ops[0]); *result = ops[0]; --ex.launches; return GPTRS_OK; }
                p.op = from == GPTRS_F32 && to == GPTRS_SI32 ? 0 : from == GPTRS_SI32 && to == GPTRS_F32 ? 1
                       : from == GPTRS_I1 && to == GPTRS_F32 ? 2 : from == GPTRS_I1 && to == GPTRS_SI32 ? 3
                       : from == GPTRS_F32 && to == GPTRS_I1 ? 4 : from == GPTRS_SI32 && to == GPTRS_I1 ? 5
                       : from == GPTRS_F32 && to == GPTRS_BF16 ? 6 : from == GPTRS_BF16 && to == GPTRS_F32 ? 7
                       : from == GPTRS_F32 && to == GPTRS_F16 ? 8 : from == GPTRS_F16 && to == GPTRS_F32 ? 9 : -1;
                if (p.op < 0) { tensor_release(out); return unimpl("cast between these dtypes"); }
                rc = launch_flat(cast_kernel, p.n, p, ex.st);
            }
            break;
        }
        case Op::Transpose: case Op::BroadcastTo: case Op::Slice: case Op::DynamicSlice: {
            if ((rc = alloc_out())) return rc;
            const auto& od = in.out.dims;
            std::vector<int64_t> istr = row_major_strides(ops[0]->dims), ostr = row_major_strides(od), use(od.size(), 0);
            int64_t off = 0;
            if (in.op == Op::Transpose) {
                if (in.a.size() != od.size()) { tensor_release(out); return spec("perm rank mismatch"); }
                for (size_t d = 0; d < od.size(); ++d) use[d] = istr[in.a[d]];
            } else if (in.op == Op::BroadcastTo) {
                const size_t shift = od.size() - ops[0]->dims.size();
                for (size_t d = 0; d < ops[0]->dims.size(); ++d) {
                    if (ops[0]->dims[d] != 1 && ops[0]->dims[d] != od[d + shift]) { tensor_release(out); return spec("shapes are not broadcast compatible"); }
                    use[d + shift] = ops[0]->dims[d] == 1 ? 0 : istr[d];
                }
            } else if (in.op == Op::Slice) {
                for (size_t d = 0; d < od.size(); ++d) {
                    if (in.a[d] + in.b[d] > ops[0]->dims[d]) { tensor_release(out); return spec("slice out of bounds"); }
                    use[d] = istr[d]; off += in.a[d] * istr[d];
                }
            } else {
                if (ops[1]->dtype != GPTRS_SI32 || ops[1]->numel() != (int64_t)od.size()) { tensor_release(out); return spec("starts must be si32[rank]"); }
                std::vector<int64_t> lim(od.size());
                for (size_t d = 0; d < od.size(); ++d) { use[d] = istr[d]; lim[d] = ops[0]->dims[d] - in.a[d]; if (lim[d] < 0) { tensor_release(out); return spec("slice larger than operand"); } }
                rc = copy_generic(ex, ops[0], out, od, use, ostr, 0, 0, static_cast<const int*>(ops[1]->data), lim, istr, false);
                break;
            }
            rc = copy_generic(ex, ops[0], out, od, use, ostr, off, 0);
            break;
        }
        case Op::DynamicUpdateSlice: {
            if ((rc = alloc_out())) return rc;
            if (ops[0]->dims != in.out.dims || ops[1]->dims.size() != in.out.dims.size() || ops[2]->dtype != GPTRS_SI32) { tensor_release(out); return spec("operand mismatch"); }
            GPTRS_CUDA_OK(cudaMemcpyAsync(out->data, ops[0]->data, out->bytes, cudaMemcpyDeviceToDevice, ex.st));
            ++ex.launches;
            std::vector<int64_t> ostr = row_major_strides(in.out.dims), ustr = row_major_strides(ops[1]->dims), lim(in.out.dims.size());
            for (size_t d = 0; d < lim.size(); ++d) { lim[d] = in.out.dims[d] - ops[1]->dims[d]; if (lim[d] < 0) { tensor_release(out); return spec("update larger than operand"); } }
            rc = copy_generic(ex, ops[1], out, ops[1]->dims, ustr, ostr, 0, 0, static_cast<const int*>(ops[2]->data), lim, ostr, true);
            break;
        }
        case Op::Concat: {
            if ((rc = alloc_out())) return rc;
            const int64_t ax = in.axis < 0 ? in.axis + (int64_t)in.out.dims.size() : in.axis;
            std::vector<int64_t> ostr = row_major_strides(in.out.dims);
            int64_t pos = 0;
            for (Tensor* t : ops) {
                if ((rc = copy_generic(ex, t, out, t->dims, row_major_strides(t->dims), ostr, 0, pos * ostr[ax]))) break;
                pos += t->dims[ax];
            }
            break;
        }
        case Op::Iota: {
            if ((rc = alloc_out())) return rc;
            if (in.out.dtype != GPTRS_SI32) { tensor_release(out); return unimpl("iota dtype other than si32"); }
            int64_t inner = 1;
            for (size_t d = in.axis + 1; d < in.out.dims.size(); ++d) inner *= in.out.dims[d];
            IotaParams p = {static_cast<int*>(out->data), n_out, inner, in.out.dims[in.axis]};
            ++ex.launches;
            rc = launch_flat(iota_kernel, n_out, p, ex.st);
            break;
        }
        case Op::Take: {
            if ((rc = alloc_out())) return rc;
            if (ops[1]->dtype != GPTRS_SI32 || dtype_size(ops[0]->dtype) != 4 || ops[0]->dims.empty()) { tensor_release(out); return spec("take needs si32 indices and a 4-byte table"); }
            const int64_t row = ops[0]->numel() / ops[0]->dims[0];
            TakeParams p = {static_cast<const uint32_t*>(ops[0]->data), static_cast<const int*>(ops[1]->data),
                            static_cast<uint32_t*>(out->data), ops[1]->numel(), row, ops[0]->dims[0], status_word()};
            ++ex.launches;
            rc = launch_flat(take_kernel, p.n_idx * row, p, ex.st);
            break;
        }
        case Op::Gather: {
            if ((rc = alloc_out())) return rc;
            const int64_t ax = in.axis < 0 ? in.axis + (int64_t)ops[0]->dims.size() : in.axis;
            if (ops[1]->dtype != GPTRS_SI32 || ops[1]->dims != in.out.dims || dtype_size(ops[0]->dtype) != 4) { tensor_release(out); return spec("gather operands"); }
            int64_t outer = 1, inner = 1;
            for (int64_t d = 0; d < ax; ++d) outer *= ops[0]->dims[d];
            for (size_t d = ax + 1; d < ops[0]->dims.size(); ++d) inner *= ops[0]->dims[d];
            GatherParams p = {static_cast<const uint32_t*>(ops[0]->data), static_cast<const int*>(ops[1]->data),
                              static_cast<uint32_t*>(out->data), outer, ops[0]->dims[ax], in.out.dims[ax], inner, status_word()};
            ++ex.launches;
            rc = launch_flat(gather_kernel, n_out, p, ex.st);
            break;
        }
        case Op::Reduce: {
            if ((rc = alloc_out())) return rc;
            if (in.a.size() != 1 || ops[0]->dtype == GPTRS_I1) { tensor_release(out); return unimpl("multi-axis or i1 reduce"); }
            const int64_t ax = in.a[0];
            ReduceParams p = {ops[0]->data, out->data, 1, ops[0]->dims[ax], 1, in.sub == "Sum" ? 0 : in.sub == "Max" ? 1 : 2,
                              ops[0]->dtype == GPTRS_SI32};
            for (int64_t d = 0; d < ax; ++d) p.outer *= ops[0]->dims[d];
            for (size_t d = ax + 1; d < ops[0]->dims.size(); ++d) p.inner *= ops[0]->dims[d];
            ++ex.launches;
            rc = launch_flat(reduce_kernel, p.outer * p.inner * 32, p, ex.st);
            break;
        }
        case Op::ReduceWindow: {
            const Tensor* X = ops[0];
            if (X->dtype != GPTRS_F32 || in.out.dtype != GPTRS_F32) return fail(GPTRS_EXECUTION, "reduce_window only supports f32 tensors");
            if (in.f0 != 0.f) return unimpl("reduce_window: accum_dtype override not supported");
            if (X->dims.size() != 4) return unimpl("reduce_window: only rank-4 tensors are supported");
            if (in.a.size() != 4 || in.b.size() != 4 || in.c.size() != 4 || in.d.size() != 4 || in.e.size() != 4)
                return fail(GPTRS_EXECUTION, "reduce_window expects window/stride/padding/dilation rank 4");
            if (in.out.dims.size() != 4) return fail(GPTRS_EXECUTION, "reduce_window output must have rank 4");
            if (in.out.dims[3] != X->dims[3]) return fail(GPTRS_EXECUTION, "reduce_window expects channels dimension preserved");
            if (in.sub != "Sum" && in.sub != "Max" && in.sub != "Min") return spec("reduce_window: unknown reduce kind");
            ReduceWindowParams p = {};
            for (int d = 0; d < 4; ++d) {
                if (in.d[d] < 1 || in.e[d] < 1 || in.b[d] < 0 || in.a[d] < 0 || X->dims[d] >= (1ll << 31) || in.out.dims[d] >= (1ll << 31))
                    return spec("reduce_window: bad window attributes");
                p.in_dims[d] = (int)X->dims[d]; p.out_dims[d] = (int)in.out.dims[d]; p.window[d] = (int)in.a[d];
                p.stride[d] = (int)in.b[d]; p.pad_lo[d] = (int)in.c[d]; p.base_dil[d] = (int)in.d[d]; p.win_dil[d] = (int)in.e[d];
            }
            if ((rc = alloc_out())) return rc;
            p.in = static_cast<const float*>(X->data); p.out = static_cast<float*>(out->data); p.n_out = in.out.numel();
            p.kind = in.sub == "Sum" ? 0 : in.sub == "Max" ? 1 : 2;
            ++ex.launches;
            rc = launch_flat(reduce_window_kernel, p.n_out, p, ex.st);
            break;
        }
        case Op::DotGeneral: {
            if ((rc = alloc_out())) return rc;
            const Tensor *A = ops[0], *B = ops[1];
            if (A->dtype != GPTRS_F32 || B->dtype != GPTRS_F32) { tensor_release(out); return unimpl("dot_general on non-f32 operands"); }
            if (in.a.size() != in.b.size() || in.c.size() != 1 || in.d.size() != 1 || in.a.size() > 1) { tensor_release(out); return unimpl("dot_general with more than one batch or contracting axis"); }
            std::vector<int64_t> as = row_major_strides(A->dims), bs = row_major_strides(B->dims);
            DotParams p = {};
            p.a = static_cast<const float*>(A->data); p.b = static_cast<const float*>(B->data); p.out = static_cast<float*>(out->data);
            p.nb = 1;
            if (!in.a.empty()) { p.nb = A->dims[in.a[0]]; p.a_sb = as[in.a[0]]; p.b_sb = bs[in.b[0]]; if (B->dims[in.b[0]] != p.nb) { tensor_release(out); return spec("batch sizes differ"); } }
            p.k = A->dims[in.c[0]]; p.a_sk = as[in.c[0]]; p.b_sk = bs[in.d[0]];
            if (B->dims[in.d[0]] != p.k) { tensor_release(out); return spec("contracting sizes differ"); }
            std::vector<int> fa, fb;
            for (int d = 0; d < (int)A->dims.size(); ++d) if ((in.a.empty() || d != in.a[0]) && d != in.c[0]) fa.push_back(d);
            for (int d = 0; d < (int)B->dims.size(); ++d) if ((in.b.empty() || d != in.b[0]) && d != in.d[0]) fb.push_back(d);
            if (fa.size() > 1 || fb.size() > 1) { tensor_release(out); return unimpl("dot_general with more than one free axis per side"); }
            p.m = fa.empty() ? 1 : A->dims[fa[0]]; p.a_sm = fa.empty() ? 0 : as[fa[0]];
            p.n = fb.empty() ? 1 : B->dims[fb[0]]; p.b_sn = fb.empty() ? 0 : bs[fb[0]];
            ++ex.launches;
            if (p.nb == 1 && p.a_sk == 1 && p.a_sm == p.k && p.b_sn == 1 && p.b_sk == p.n)
                rc = gptrs_cuda_matmul_f32(p.a, p.b, p.out, p.m, p.n, p.k, nullptr, nullptr, 0, ex.st);  // [M,K].[K,N]
            else
                rc = launch_flat(dot_kernel, p.nb * p.m * p.n, p, ex.st);
            break;
        }
        case Op::FusedLayerNorm: case Op::FusedRmsNorm: {
            if ((rc = alloc_out())) return rc;
            const int64_t d = in.out.dims.back(), rows = n_out / d;
            ++ex.launches;
            // the fused kernels take the row in `hidden` without modifying it when no delta is given
            rc = in.op == Op::FusedLayerNorm
                     ? gptrs_cuda_add_layer_norm(static_cast<float*>(ops[0]->data), nullptr, GPTRS_F32, nullptr, static_cast<const float*>(ops[1]->data),
                                                 static_cast<const float*>(ops[2]->data), in.f0, out->data, GPTRS_F32, nullptr, nullptr, rows, d, ex.st)
                     : gptrs_cuda_add_rms_norm(static_cast<float*>(ops[0]->data), nullptr, GPTRS_F32, static_cast<const float*>(ops[1]->data), in.f0,
                                               out->data, GPTRS_F32, nullptr, rows, d, ex.st);
            break;
        }
        case Op::FusedSoftmax: {
            if ((rc = alloc_out())) return rc;
            const int64_t d = in.out.dims.back();
            ++ex.launches;
            rc = gptrs_cuda_softmax_last_dim(static_cast<const float*>(ops[0]->data), static_cast<float*>(out->data), n_out / d, d, ex.st);
            break;
        }
        case Op::FusedGelu: {
            if ((rc = alloc_out())) return rc;
            ++ex.launches;
            rc = gptrs_cuda_gelu(static_cast<const float*>(ops[0]->data), static_cast<float*>(out->data), n_out, ex.st);
            break;
        }
        case Op::FusedMatmulBias: {   // in.axis = 1: GELU on the sum
            if ((rc = alloc_out())) return rc;
            ++ex.launches;
            rc = gptrs_cuda_matmul_f32(static_cast<const float*>(ops[0]->data), static_cast<const float*>(ops[1]->data), static_cast<float*>(out->data),
                                       ops[0]->dims[0], ops[1]->dims[1], ops[0]->dims[1], static_cast<const float*>(ops[2]->data), nullptr,
                                       in.axis == 1 ? 1 : 0, ex.st);
            break;
        }
        case Op::FusedAttentionDecode: {
            if ((rc = alloc_out())) return rc;
            static int* zero_slot = nullptr;  // the cache operands hold ONE sequence: row 0
            if (!zero_slot) {
                if (cudaMalloc(&zero_slot, sizeof(int)) != cudaSuccess) { tensor_release(out); return fail(GPTRS_EXECUTION, "cudaMalloc failed"); }
                cudaMemset(zero_slot, 0, sizeof(int));
            }
            ++ex.launches;
            // q [Hq,1,hd] is read as the Q part of one packed row; the position is clamped on the device like the
            // DynamicSlice it replaces
            rc = gptrs_cuda_attention_decode_f32(static_cast<const float*>(ops[0]->data), static_cast<const float*>(ops[1]->data),
                                                 static_cast<const float*>(ops[2]->data), static_cast<const int32_t*>(ops[3]->data), zero_slot,
                                                 static_cast<float*>(out->data), 1, in.a[0], in.a[1], in.a[2], in.a[3], ex.st);
            break;
        }
        case Op::Dequantize: {
            // canonical W8 (si8 [N][K], fp16 scales [N]) or W4 (two si4 per byte [N][K/2], fp16 scales [N][K/128]) -> f32 [N][K]
            if ((rc = alloc_out())) return rc;
            const int64_t N = in.out.dims[0], K = in.out.dims[1];
            ++ex.launches;
            rc = ops[0]->dtype == GPTRS_SI8
                     ? gptrs_cuda_dequantize_w8(static_cast<const int8_t*>(ops[0]->data), static_cast<const uint16_t*>(ops[1]->data), K, N, 1,
                                                static_cast<float*>(out->data), ex.st)
                     : gptrs_cuda_dequantize_w4(static_cast<const uint8_t*>(ops[0]->data), static_cast<const uint16_t*>(ops[1]->data), K, N, 1,
                                                static_cast<float*>(out->data), ex.st);
            break;
        }
        case Op::FusedQuantMatmul: {
            // x f32 [M][K] . dequant(q, scales)^T -> f32 [M][N] on the quantised matmul kernels. The kernel layout of the
            // weight is derived once per weight handle and kept with it (the derived-parameter memo of the reference's
            // resolver, crates/gpt-rs/src/backend/param_resolver.rs:11-50, keyed here by the handle itself).
            Tensor *X = ops[0], *Q = ops[1], *S = ops[2];
            const bool w8 = Q->dtype == GPTRS_SI8;
            const int64_t M = X->dims[0], K = X->dims[1], N = Q->dims[0];
            const size_t need = w8 ? gptrs_cuda_w8a16_packed_bytes(N, K) : gptrs_cuda_w4a16_packed_bytes(N, K);
            if (need == 0) return spec("quantised matmul needs K % 128 == 0 and N % 16 == 0");
            static std::mutex derive_mu;
            Tensor* packed = nullptr;
            {
                std::lock_guard<std::mutex> lk(derive_mu);
                if (!Q->derived || Q->derived_with != S->data || Q->derived->bytes != need) {
                    Tensor* fresh = nullptr;
                    int64_t pd[1] = {(int64_t)need};
                    if ((rc = tensor_alloc(GPTRS_UI8, 1, pd, false, &fresh))) return rc;
                    rc = w8 ? gptrs_cuda_w8a16_repack(static_cast<const int8_t*>(Q->data), static_cast<const uint16_t*>(S->data), N, K, 0, fresh->data, ex.st)
                            : gptrs_cuda_w4a16_repack(static_cast<const uint8_t*>(Q->data), static_cast<const uint16_t*>(S->data), N, K, 0, fresh->data, ex.st);
                    if (rc) { tensor_release(fresh); return rc; }
                    ex.launches += 2;
                    tensor_release(Q->derived);
                    Q->derived = fresh;
                    Q->derived_with = S->data;
                }
                packed = Q->derived;
                tensor_retain(packed);
            }
            Tensor* xb = nullptr;   // the kernels take bf16 activations
            if (ex.arena && ex.arena_off >= 0) {   // planned: right behind the result
                const int64_t main_bytes = (((int64_t)in.out.numel() * (int64_t)dtype_size(in.out.dtype)) + 255) & ~(int64_t)255;
                xb = new Tensor();
                xb->dtype = GPTRS_BF16; xb->dims = X->dims;
                xb->bytes = (size_t)X->numel() * 2;
                xb->data = static_cast<unsigned char*>(ex.arena->data) + ex.arena_off + main_bytes;
                xb->owns = false; xb->base = ex.arena; xb->device = ex.arena->device;
                tensor_retain(ex.arena);
            } else if ((rc = tensor_alloc(GPTRS_BF16, 2, X->dims.data(), false, &xb))) { tensor_release(packed); return rc; }
            EwParams cp = {};
            cp.a = X->data; cp.out = xb->data; cp.n = X->numel(); cp.op = 6;
            rc = launch_flat(cast_kernel, cp.n, cp, ex.st);
            if (!rc) rc = alloc_out();
            if (!rc) {
                gptrs_matmul_epilogue ep = {};
                ep.out_dtype = GPTRS_F32;
                rc = w8 ? gptrs_cuda_quant_matmul_w8a16(xb->data, packed->data, out->data, M, N, K, &ep, ex.st)
                        : gptrs_cuda_quant_matmul_w4a16(xb->data, packed->data, out->data, M, N, K, &ep, ex.st);
            }
            ex.launches += 2;
            // the temporaries are read by kernels already enqueued on this stream; their memory is pooled and handed out
            // again only to work enqueued later on a stream (run_program is synchronous at its end)
            tensor_release(xb);
            tensor_release(packed);
            break;
        }
        case Op::FusedAddRmsNorm: case Op::FusedAddLayerNorm: {
            // (residual, update, gamma[, beta]) -> norm(residual + update); with a second result the sum is written too
            if ((rc = alloc_out())) return rc;
            const bool ln = in.op == Op::FusedAddLayerNorm;
            const int64_t d = in.out.dims.back(), rows = n_out / d;
            Tensor* sum = nullptr;
            if (in.side_id && ex.arena && ex.arena_off >= 0) {   // planned: right behind the first result
                const int64_t main_bytes = (((int64_t)in.out.numel() * (int64_t)dtype_size(in.out.dtype)) + 255) & ~(int64_t)255;
                sum = new Tensor();
                sum->dtype = in.side_out.dtype; sum->dims = in.side_out.dims;
                sum->bytes = (size_t)in.side_out.numel() * dtype_size(in.side_out.dtype);
                sum->data = static_cast<unsigned char*>(ex.arena->data) + ex.arena_off + main_bytes;
                sum->owns = false; sum->base = ex.arena; sum->device = ex.arena->device;
                tensor_retain(ex.arena);
            } else if (in.side_id && (rc = tensor_alloc(in.side_out.dtype, (int)in.side_out.dims.size(), in.side_out.dims.data(), false, &sum))) break;
            ++ex.launches;
            rc = add_norm_out_of_place(static_cast<const float*>(ops[0]->data), static_cast<const float*>(ops[1]->data),
                                       sum ? static_cast<float*>(sum->data) : nullptr, static_cast<const float*>(ops[2]->data),
                                       ln ? static_cast<const float*>(ops[3]->data) : nullptr, in.f0, static_cast<float*>(out->data), rows, d, ln, ex.st);
            if (rc) tensor_release(sum); else ex.side = sum;
            break;
        }
        case Op::CustomCall:
            return fail(GPTRS_UNIMPLEMENTED, "custom_call target '" + in.sub + "' is not implemented by the cuda backend");
        default:
            return unimpl("operation outside the decode-path subset of this backend");
    }
    if (rc) { tensor_release(out); return rc; }
    *result = out;
    return GPTRS_OK;
}

}  // namespace
}  // namespace ptir
}  // namespace gptrs

using namespace gptrs;
using namespace gptrs::ptir;

extern "C" {

namespace {

// The cached plan of a program text on the current device (parsed, verified, rewritten, buffers planned).
int plan_for(const char* program_json, size_t len, std::shared_ptr<Plan>* out) {
    const int device = current_device();
    const uint64_t key = fnv1a(program_json, len) ^ (g_fusion_enabled ? 0 : 0x5bd1e995u) ^ ((uint64_t)(device + 1) * 0x9e3779b97f4a7c15ull);
    std::shared_ptr<Plan> plan;
    {
        std::lock_guard<std::mutex> lk(g_plan_mu);
        auto it = g_plans.find(key);
        if (it != g_plans.end()) { plan = it->second; ++g_plan_hits; }
    }
    if (!plan) {
        Json root;
        std::string err;
        if (!parse_json(program_json, len, &root, &err)) return fail(GPTRS_SPEC_VIOLATION, "program json: " + err);
        auto p = std::make_shared<Plan>();
        int st = build_function(root, &p->fn, &err);
        if (!st) st = verify_function(p->fn, &err);   // before any launch: arity, attribute ranges, declared result types
        if (st) return fail(st == 2 ? GPTRS_UNIMPLEMENTED : GPTRS_SPEC_VIOLATION, err);
        if (g_fusion_enabled) rewrite(*p); else count_uses(*p);
        if (int rc = upload_literals(*p)) return rc;
        p->device = device;
        count_uses(*p);
        if (g_arena_enabled) plan_buffers(*p);
        std::lock_guard<std::mutex> lk(g_plan_mu);
        g_plans[key] = p;
        ++g_plan_builds;
        plan = p;
    }
    *out = plan;
    return GPTRS_OK;
}

// The instructions of the plan, launched on `st` (directly or into a stream capture). Fills outputs (retained).
int run_instructions(Plan& pl, gptrs_tensor* const* inputs, size_t n_inputs, gptrs_tensor** outputs, cudaStream_t st, int64_t* launches) {
    const Function& fn = pl.fn;
    Exec ex;
    ex.st = st;
    ex.arena = pl.arena;
    for (size_t i = 0; i < n_inputs; ++i) {
        Tensor* t = reinterpret_cast<Tensor*>(inputs[i]);
        tensor_retain(t);
        ex.env[fn.param_ids[i]] = t;
    }
    for (size_t ii = 0; ii < fn.body.size(); ++ii) {
        const Inst& in = fn.body[ii];
        if (in.dead) continue;
        std::vector<Tensor*> ops(in.operands.size(), nullptr);
        int rc = GPTRS_OK;
        for (size_t i = 0; i < ops.size() && !rc; ++i) rc = ex.value(in.operands[i], &ops[i]);
        Tensor* res = nullptr;
        ex.arena_off = ii < pl.arena_offset.size() ? pl.arena_offset[ii] : -1;
        ex.side = nullptr;
        if (!rc) rc = exec_inst(ex, in, ops, &res);
        for (Tensor* t : ops) tensor_release(t);
        if (rc) return rc;
        if (ex.side) { ex.env[in.side_id] = ex.side; ex.side = nullptr; }
        if (res->dtype != in.out.dtype || res->dims != in.out.dims) {
            tensor_release(res);
            return fail(GPTRS_SPEC_VIOLATION, in.name + " (%" + std::to_string(in.id) + ") produced a value that does not match its declared type");
        }
        ex.env[in.id] = res;
    }
    for (size_t i = 0; i < fn.result_ids.size(); ++i) {
        auto it = ex.env.find(fn.result_ids[i]);
        if (it == ex.env.end()) return fail(GPTRS_SPEC_VIOLATION, "result value is undefined");
        tensor_retain(it->second);
        outputs[i] = reinterpret_cast<gptrs_tensor*>(it->second);
    }
    *launches = ex.launches;
    return GPTRS_OK;
}

std::atomic<int> g_plan_graphs{1};   // gptrs_cuda_set_plan_graphs
std::atomic<int> g_plan_graph_pdl{[] { const char* e = getenv("GPTRS_PLAN_GRAPH_PDL"); return (e && e[0] == '0') ? 0 : 1; }()};
thread_local int64_t g_last_graph_replays = 0;

// Replay: take the results from the pool in the recorded order; launch the graph whose blocks they are.
bool try_replay(Plan& pl, gptrs_tensor* const* inputs, size_t n_inputs, gptrs_tensor** outputs, cudaStream_t st, int64_t* launches) {
    for (auto& g : pl.graphs) {
        bool same = g.in_ptrs.size() == n_inputs;
        for (size_t i = 0; i < n_inputs && same; ++i) same = reinterpret_cast<Tensor*>(inputs[i])->data == g.in_ptrs[i];
        if (!same) continue;
        std::vector<Tensor*> got;
        bool ok = true;
        for (size_t k = 0; k < g.allocs.size() && ok; ++k) {
            Tensor* t = nullptr;
            if (tensor_alloc(g.allocs[k].dtype, (int)g.allocs[k].dims.size(), g.allocs[k].dims.data(), false, &t) != GPTRS_OK) { ok = false; break; }
            got.push_back(t);
            ok = t->data == g.alloc_ptrs[k];
        }
        if (ok && cudaGraphLaunch(g.exec, st) == cudaSuccess) {
            for (size_t i = 0; i < g.result_of.size(); ++i) outputs[i] = reinterpret_cast<gptrs_tensor*>(got[g.result_of[i]]);
            *launches = g.launches;
            return true;
        }
        // the pool handed out other blocks: give them back in reverse order, so that the pool's stacks are as before
        for (size_t k = got.size(); k-- > 0;) tensor_release(got[k]);
        cudaGetLastError();
    }
    return false;
}

// One execution recorded into a graph. Returns false (with nothing launched and nothing kept) when the execution does
// not fit the scheme: then the caller runs it kernel by kernel.
bool capture_run(Plan& pl, gptrs_tensor* const* inputs, size_t n_inputs, gptrs_tensor** outputs, cudaStream_t st, int64_t* launches, int* rc_out) {
    const size_t n_res = pl.fn.result_ids.size();
    std::vector<Tensor*> record;
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed) != cudaSuccess) { cudaGetLastError(); return false; }
    g_alloc_record = &record;
    // recorded with programmatic dependent launch edges, like the engine's decode step: every kernel of the library waits
    // (griddepcontrol.wait) before it reads what its predecessor wrote, so set-up and scheduling of a kernel overlap the
    // one in front
    const int pdl_before = g_use_pdl;
    g_use_pdl = g_plan_graph_pdl.load(std::memory_order_relaxed) ? 1 : pdl_before;
    int rc = run_instructions(pl, inputs, n_inputs, outputs, st, launches);
    g_use_pdl = pdl_before;
    g_alloc_record = nullptr;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(st, &graph);
    auto drop_outputs = [&]() { if (!rc) for (size_t i = 0; i < n_res; ++i) tensor_release(reinterpret_cast<Tensor*>(outputs[i])); };
    if (getenv("GPTRS_DEBUG_GRAPH") && (rc || e != cudaSuccess)) fprintf(stderr, "plan graph: capture failed rc=%d cuda=%s\n", rc, cudaGetErrorString(e));
    if (rc || e != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        drop_outputs();
        if (rc) { *rc_out = rc; return true; }   // a real error of the program: report it
        return false;
    }
    // fits only if every allocation of the run is exactly one result and no result is an input or a view
    Plan::RunGraph g;
    bool fits = record.size() == n_res;
    g.result_of.assign(n_res, -1);
    for (size_t i = 0; i < n_res && fits; ++i) {
        Tensor* t = reinterpret_cast<Tensor*>(outputs[i]);
        for (size_t k = 0; k < record.size(); ++k) if (record[k] == t) g.result_of[i] = (int)k;
        fits = g.result_of[i] >= 0;
        for (size_t j = 0; j < i && fits; ++j) fits = g.result_of[j] != g.result_of[i];
    }
    if (getenv("GPTRS_DEBUG_GRAPH")) {
        fprintf(stderr, "plan graph: %zu allocations for %zu results, fits=%d\n", record.size(), n_res, (int)fits);
        if (!fits) for (Tensor* t : record) {
            bool is_res = false;
            for (size_t i = 0; i < n_res; ++i) is_res = is_res || reinterpret_cast<Tensor*>(outputs[i]) == t;
            if (!is_res) fprintf(stderr, "  extra allocation: dtype %d, %zu bytes, rank %zu\n", t->dtype, t->bytes, t->dims.size());
        }
    }
    if (fits) {
        e = cudaGraphInstantiate(&g.exec, graph, 0);
        fits = e == cudaSuccess;
    }
    cudaGraphDestroy(graph);
    if (fits) fits = cudaGraphLaunch(g.exec, st) == cudaSuccess;
    if (!fits) {
        if (g.exec) cudaGraphExecDestroy(g.exec);
        cudaGetLastError();
        drop_outputs();
        return false;
    }
    for (size_t i = 0; i < n_inputs; ++i) g.in_ptrs.push_back(reinterpret_cast<Tensor*>(inputs[i])->data);
    for (Tensor* t : record) {
        TSpec sp;
        sp.dtype = t->dtype;
        sp.dims = t->dims;
        g.allocs.push_back(sp);
        g.alloc_ptrs.push_back(t->data);
    }
    g.launches = *launches;
    pl.graphs.push_back(std::move(g));
    return true;
}

int execute_plan(const std::shared_ptr<Plan>& plan, gptrs_tensor* const* inputs, size_t n_inputs, gptrs_tensor** outputs,
                 size_t outputs_cap, size_t* n_outputs, void* stream) {
    const Function& fn = plan->fn;
    if (plan->device != current_device()) return fail(GPTRS_SPEC_VIOLATION, "the program was prepared on another device");
    GPTRS_REQUIRE(n_inputs == fn.param_ids.size(), "entry input count does not match the function parameters");
    GPTRS_REQUIRE(n_outputs && outputs_cap >= fn.result_ids.size() && (outputs || fn.result_ids.empty()), "output array too small");
    // one execution at a time per plan: the temporaries of the function live at fixed offsets of the plan's arena
    std::lock_guard<std::mutex> run_lock(plan->run_mu);
    if (plan->arena_bytes > 0 && !plan->arena) {
        int64_t ad[1] = {plan->arena_bytes};
        if (int rc = tensor_alloc(GPTRS_UI8, 1, ad, false, &plan->arena)) return rc;
    }
    for (size_t i = 0; i < n_inputs; ++i) {
        Tensor* t = reinterpret_cast<Tensor*>(inputs[i]);
        GPTRS_REQUIRE(t, "null input handle");
        if (t->dtype != fn.params[i].dtype || t->dims != fn.params[i].dims)
            return fail(GPTRS_SPEC_VIOLATION, "input " + std::to_string(i) + " does not match the declared parameter type");
    }
    cudaStream_t st = as_stream(stream);
    struct { int64_t launches = 0; } ex;
    bool done = false;
    g_last_graph_replays = 0;
    // The first two executions run kernel by kernel (they fill the memos of derived weight layouts); later ones replay a
    // graph when one fits, and record one (at most four per plan) when none does.
    const bool graphs_on = g_plan_graphs.load(std::memory_order_relaxed) != 0 && plan->graph_ok && plan->arena && !fn.result_ids.empty();
    ++plan->runs;
    if (graphs_on && plan->runs > 2) {
        if (!plan->side_stream) {
            if (cudaStreamCreateWithFlags(&plan->side_stream, cudaStreamNonBlocking) != cudaSuccess ||
                cudaEventCreateWithFlags(&plan->ev_in, cudaEventDisableTiming) != cudaSuccess ||
                cudaEventCreateWithFlags(&plan->ev_out, cudaEventDisableTiming) != cudaSuccess) {
                cudaGetLastError();
                plan->graph_ok = false;
            }
        }
        if (plan->graph_ok) {
            cudaStream_t gs = plan->side_stream;
            GPTRS_CUDA_OK(cudaEventRecord(plan->ev_in, st));
            GPTRS_CUDA_OK(cudaStreamWaitEvent(gs, plan->ev_in, 0));
            done = try_replay(*plan, inputs, n_inputs, outputs, gs, &ex.launches);
            if (done) g_last_graph_replays = 1;
            if (!done && plan->graphs.size() < 4) {
                int rc = GPTRS_OK;
                done = capture_run(*plan, inputs, n_inputs, outputs, gs, &ex.launches, &rc);
                if (done && rc) return rc;
                if (!done && ++plan->graph_failures >= 2) plan->graph_ok = false;
            }
            if (done) {
                GPTRS_CUDA_OK(cudaEventRecord(plan->ev_out, gs));
                GPTRS_CUDA_OK(cudaStreamWaitEvent(st, plan->ev_out, 0));
            }
        }
    }
    if (!done) {
        int rc = run_instructions(*plan, inputs, n_inputs, outputs, st, &ex.launches);
        if (rc) return rc;
    }
    cudaStream_t ex_st = st;
    *n_outputs = fn.result_ids.size();
    g_last_launches = ex.launches;
    g_last_fused = plan->fused;
    // report a device-side index error (take / gather) the way ref-cpu reports it: as an error
    int* sw = status_word();
    if (sw) {
        int hs = 0;
        GPTRS_CUDA_OK(cudaMemcpyAsync(&hs, sw, 4, cudaMemcpyDeviceToHost, ex_st));
        GPTRS_CUDA_OK(cudaStreamSynchronize(ex_st));
        if (hs) {
            cudaMemsetAsync(sw, 0, 4, ex_st);
            for (size_t i = 0; i < fn.result_ids.size(); ++i) tensor_release(reinterpret_cast<Tensor*>(outputs[i]));
            *n_outputs = 0;
            return fail(GPTRS_EXECUTION, "index out of range in take/gather");
        }
    }
    return GPTRS_OK;
}

}  // namespace

int gptrs_cuda_run_program(const char* program_json, size_t len, gptrs_tensor* const* inputs, size_t n_inputs,
                           gptrs_tensor** outputs, size_t outputs_cap, size_t* n_outputs, void* stream) {
    GPTRS_REQUIRE(program_json && n_outputs && (n_inputs == 0 || inputs), "null pointer");
    std::shared_ptr<Plan> plan;
    if (int rc = plan_for(program_json, len, &plan)) return rc;
    return execute_plan(plan, inputs, n_inputs, outputs, outputs_cap, n_outputs, stream);
}

int gptrs_cuda_program_prepare(const char* program_json, size_t len, gptrs_program** out) {
    GPTRS_REQUIRE(program_json && out, "null pointer");
    std::shared_ptr<Plan> plan;
    if (int rc = plan_for(program_json, len, &plan)) return rc;
    *out = reinterpret_cast<gptrs_program*>(new std::shared_ptr<Plan>(plan));
    return GPTRS_OK;
}

int gptrs_cuda_program_run(gptrs_program* program, gptrs_tensor* const* inputs, size_t n_inputs, gptrs_tensor** outputs,
                           size_t outputs_cap, size_t* n_outputs, void* stream) {
    GPTRS_REQUIRE(program && n_outputs && (n_inputs == 0 || inputs), "null pointer");
    {
        std::lock_guard<std::mutex> lk(g_plan_mu);
        ++g_plan_hits;
    }
    return execute_plan(*reinterpret_cast<std::shared_ptr<Plan>*>(program), inputs, n_inputs, outputs, outputs_cap, n_outputs, stream);
}

void gptrs_cuda_program_release(gptrs_program* program) { delete reinterpret_cast<std::shared_ptr<Plan>*>(program); }

int gptrs_cuda_execute_instruction(const char* instruction_json, size_t len, gptrs_tensor* const* inputs, size_t n_inputs,
                                   gptrs_tensor** outputs, size_t outputs_cap, size_t* n_outputs, void* stream) {
    GPTRS_REQUIRE(instruction_json && n_outputs && (n_inputs == 0 || inputs), "null pointer");
    Json inst;
    std::string err;
    if (!parse_json(instruction_json, len, &inst, &err)) return fail(GPTRS_SPEC_VIOLATION, "instruction json: " + err);
    const Json *id = inst.get("id"), *operands = inst.get("operands");
    if (!id || !operands || operands->kind != Json::Array) return fail(GPTRS_SPEC_VIOLATION, "malformed instruction");
    GPTRS_REQUIRE(n_inputs == operands->arr.size(), "one input handle per operand is expected");
    // A one-instruction function around the text as given: each distinct operand value becomes a parameter typed by
    // the handle passed for it; literal operands stay literals (their handle is not read).
    static const char* const kNames[] = {"F32", "F16", "Bf16", "Si32", "I1", "Si8", "Ui8"};  // gptrs_dtype order
    std::string params, pids;
    std::vector<gptrs_tensor*> args;
    std::vector<int64_t> seen;
    for (size_t i = 0; i < operands->arr.size(); ++i) {
        const Json* v = operands->arr[i].get("Value");
        if (!v) continue;
        const int64_t vid = v->as_int();
        bool dup = false;
        for (int64_t s2 : seen) dup = dup || s2 == vid;
        if (dup) continue;
        const Tensor* t = reinterpret_cast<const Tensor*>(inputs[i]);
        GPTRS_REQUIRE(t, "null input handle");
        GPTRS_REQUIRE(t->dtype >= 0 && t->dtype < 7, "input handle of an unknown dtype");
        seen.push_back(vid);
        args.push_back(inputs[i]);
        if (!params.empty()) { params += ","; pids += ","; }
        params += std::string("{\"Tensor\":{\"dtype\":\"") + kNames[t->dtype] + "\",\"shape\":{\"dims\":[";
        for (size_t d = 0; d < t->dims.size(); ++d) params += (d ? ",{\"Static\":" : "{\"Static\":") + std::to_string(t->dims[d]) + "}";
        params += "]}}}";
        pids += std::to_string(vid);
    }
    std::string text = "{\"spec_version\":\"ptir.v0.4\",\"entry\":\"instruction\",\"functions\":[{\"name\":\"instruction\",\"parameters\":[" +
                       params + "],\"parameter_ids\":[" + pids + "],\"results\":[],\"body\":[";
    text.append(instruction_json, len);
    text += "],\"hints\":[],\"result_ids\":[" + std::to_string(id->as_int()) + "]}],\"regions\":[]}";
    return gptrs_cuda_run_program(text.data(), text.size(), args.data(), args.size(), outputs, outputs_cap, n_outputs, stream);
}

namespace {

Json jnum(double v) { Json j; j.kind = Json::Number; j.num = v; return j; }
Json jstr(const std::string& v) { Json j; j.kind = Json::String; j.str = v; return j; }
Json jobj(std::vector<std::pair<std::string, Json>> kv) { Json j; j.kind = Json::Object; j.obj = std::move(kv); return j; }
Json jarr(std::vector<Json> v) { Json j; j.kind = Json::Array; j.arr = std::move(v); return j; }

Json tensor_spec_json(const TSpec& t) {
    static const char* const kNames[] = {"F32", "F16", "Bf16", "Si32", "I1", "Si8", "Ui8"};  // gptrs_dtype order
    std::vector<Json> dims;
    for (int64_t d : t.dims) dims.push_back(jobj({{"Static", jnum((double)d)}}));
    return jobj({{"dtype", jstr(kNames[t.dtype])}, {"shape", jobj({{"dims", jarr(std::move(dims))}})}});
}

// A fused operation as the CustomCall instruction the reference's rewriters would insert (docs/backend.md:568-592).
Json fused_instruction_json(const Inst& in) {
    std::vector<Json> operands;
    for (const Operand& o : in.operands) {
        if (!o.is_literal) { operands.push_back(jobj({{"Value", jnum(o.id)}})); continue; }
        std::vector<Json> bytes;
        for (uint8_t b : o.bytes) bytes.push_back(jnum(b));
        operands.push_back(jobj({{"Literal", jobj({{"spec", tensor_spec_json(o.lit)}, {"bytes", jarr(std::move(bytes))}})}}));
    }
    std::vector<std::pair<std::string, Json>> attrs;
    // CustomCallAttr is adjacently tagged (#[serde(tag = "kind", content = "value")], spec.rs:602-613)
    if (in.op == Op::FusedLayerNorm || in.op == Op::FusedRmsNorm || in.op == Op::FusedAddRmsNorm || in.op == Op::FusedAddLayerNorm)
        attrs.push_back({"eps", jobj({{"kind", jstr("F64")}, {"value", jnum((double)in.f0)}})});
    if (in.op == Op::FusedMatmulBias && in.axis == 1) attrs.push_back({"activation", jobj({{"kind", jstr("String")}, {"value", jstr("gelu")}})});
    if (in.op == Op::FusedQuantMatmul) attrs.push_back({"group_size", jobj({{"kind", jstr("I64")}, {"value", jnum(in.sub == "w4" ? 128 : 0)}})});
    if (in.op == Op::FusedAttentionDecode) {
        std::vector<Json> g;
        for (int64_t v : in.a) g.push_back(jnum((double)v));
        attrs.push_back({"geometry", jobj({{"kind", jstr("I64Array")}, {"value", jarr(std::move(g))}})});
    }
    const std::string target = in.op == Op::FusedQuantMatmul ? (in.sub == "w8" ? "gpt_rs.cuda.quant_matmul_w8a16.v1" : "gpt_rs.cuda.quant_matmul_w4a16.v1")
                                                             : std::string(fused_target(in.op));
    Json call = jobj({{"CustomCall", jobj({{"target", jstr(target)}, {"attrs", jobj(std::move(attrs))}})}});
    return jobj({{"id", jnum(in.id)}, {"op", std::move(call)}, {"operands", jarr(std::move(operands))},
                 {"output", jobj({{"Tensor", tensor_spec_json(in.out)}})}});
}

}  // namespace

int gptrs_cuda_pipeline_fuse(const char* program_json, size_t len, char* out, size_t out_cap, size_t* written, int64_t* n_fused) {
    GPTRS_REQUIRE(program_json && written, "null pointer");
    Json root;
    std::string err;
    if (!parse_json(program_json, len, &root, &err)) return fail(GPTRS_SPEC_VIOLATION, "program json: " + err);
    Plan plan;
    int st = build_function(root, &plan.fn, &err);
    if (!st) st = verify_function(plan.fn, &err);
    if (st) return fail(st == 2 ? GPTRS_UNIMPLEMENTED : GPTRS_SPEC_VIOLATION, err);
    rewrite(plan, false);
    // the entry function's body: surviving instructions as they were, fused ones as CustomCalls, in the old order
    const std::string entry = root.get("entry")->str;
    for (auto& kv : root.obj) {
        if (kv.first != "functions") continue;
        for (Json& f : kv.second.arr) {
            const Json* name = f.get("name");
            if (!name || name->str != entry) continue;
            for (auto& fkv : f.obj) {
                if (fkv.first != "body") continue;
                std::vector<Json> body;
                for (const Inst& in : plan.fn.body) {
                    if (in.dead) continue;
                    if (fused_target(in.op) || in.op == Op::FusedQuantMatmul) body.push_back(fused_instruction_json(in));
                    else body.push_back(fkv.second.arr[in.src]);
                }
                fkv.second.arr = std::move(body);
            }
        }
    }
    std::string text;
    write_json(root, &text);
    *written = text.size();
    if (n_fused) *n_fused = plan.fused;
    if (out && out_cap >= text.size()) memcpy(out, text.data(), text.size());
    return GPTRS_OK;
}

int gptrs_cuda_verify_program(const char* program_json, size_t len) {
    GPTRS_REQUIRE(program_json, "null pointer");
    Json root;
    std::string err;
    if (!parse_json(program_json, len, &root, &err)) return fail(GPTRS_SPEC_VIOLATION, "program json: " + err);
    Function fn;
    int st = build_function(root, &fn, &err);
    if (!st) st = verify_function(fn, &err);
    if (st) return fail(st == 2 ? GPTRS_UNIMPLEMENTED : GPTRS_SPEC_VIOLATION, err);
    return GPTRS_OK;
}

int gptrs_cuda_run_program_stats(int64_t* plan_builds, int64_t* plan_hits, int64_t* last_launches, int64_t* last_fused) {
    if (plan_builds) *plan_builds = g_plan_builds;
    if (plan_hits) *plan_hits = g_plan_hits;
    if (last_launches) *last_launches = g_last_launches;
    if (last_fused) *last_fused = g_last_fused;
    return GPTRS_OK;
}

int gptrs_cuda_set_fusion(int enabled) {
    g_fusion_enabled = enabled ? 1 : 0;
    return GPTRS_OK;
}

int gptrs_cuda_set_plan_graphs(int enabled) {
    g_plan_graphs.store(enabled ? 1 : 0);
    return GPTRS_OK;
}

int gptrs_cuda_last_run_replayed_graph(void) { return (int)g_last_graph_replays; }

int gptrs_cuda_set_buffer_plan(int enabled) {
    g_arena_enabled = enabled ? 1 : 0;
    std::lock_guard<std::mutex> lk(g_plan_mu);
    g_plans.clear();   // plans are built with or without an arena
    return GPTRS_OK;
}

int gptrs_cuda_pipeline(const char* phase, const char* program_json, size_t len, char* out, size_t out_cap, size_t* written,
                        int64_t* n_rewrites) {
    GPTRS_REQUIRE(phase && program_json && written, "null pointer");
    const std::string ph = phase;
    if (ph == "pre" || ph == "fuse") return gptrs_cuda_pipeline_fuse(program_json, len, out, out_cap, written, n_rewrites);
    if (ph != "legalize" && ph != "cleanup") return fail(GPTRS_SPEC_VIOLATION, "unknown pipeline phase '" + ph + "' (pre, legalize, fuse, cleanup)");
    // legalize: every operation of the decode-path subset runs as written, nothing to lower. cleanup: the rewrites
    // sweep their own dead instructions. Both return the program unchanged (after checking that it parses and verifies).
    int rc = gptrs_cuda_verify_program(program_json, len);
    if (rc) return rc;
    *written = len;
    if (n_rewrites) *n_rewrites = 0;
    if (out && out_cap >= len) memcpy(out, program_json, len);
    return GPTRS_OK;
}

}  // extern "C"
