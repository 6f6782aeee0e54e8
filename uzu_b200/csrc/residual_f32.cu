// Glue kernels of the parallel-block family (f32 residual stream): grouped RMS norm, embedding rows into f32, the clamped gated unit,
// tanh, residual add, logit cap, and the table router (expert-sorted pair lists + weighted combine). Everything is f32 arithmetic.
#include "common.cuh"

namespace uzu {

// one CTA per (row, group); a thread keeps up to 8 of the part's elements in registers between the sum and the scaling
__global__ void __launch_bounds__(256) group_rms_norm_kernel(const uzu_group_rms_norm_args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[32];
    const uint32_t row = blockIdx.x, g = blockIdx.y;
    const uint32_t src = a.row_indices ? reinterpret_cast<const uint32_t*>(a.row_indices)[row] : row;
    const uint32_t part = a.n / a.groups, base = g * part;
    const float* in = reinterpret_cast<const float*>(a.input) + (size_t)src * a.in_stride + base;
    float* out = reinterpret_cast<float*>(a.output) + (size_t)row * a.out_stride + base;
    const float* sc = a.scales ? reinterpret_cast<const float*>(a.scales) + base : nullptr;
    constexpr int KEEP = 8;
    float v[KEEP];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        v[j] = i < part ? in[i] : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < KEEP; ++j) ss = fmaf(v[j], v[j], ss);
    for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < part; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)part + a.epsilon);
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const uint32_t i = threadIdx.x + j * blockDim.x;
        if (i < part) out[i] = sc ? v[j] * inv * sc[i] : v[j] * inv;
    }
    for (uint32_t i = threadIdx.x + KEEP * blockDim.x; i < part; i += blockDim.x) out[i] = sc ? in[i] * inv * sc[i] : in[i] * inv;
}

template <typename TW>
__global__ void embedding_f32_kernel(const uint32_t* tokens, const TW* table, float* out, uint32_t vocab, uint32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t row = blockIdx.y;
    const uint32_t tok = tokens[row];
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = 0.0f;
    if (tok < vocab) {
        if constexpr (sizeof(TW) == 2) v = __bfloat162float(table[(size_t)tok * n + i]);
        else v = table[(size_t)tok * n + i];
    }
    out[(size_t)row * n + i] = v;
}

__global__ void clamped_glu_kernel(const float* gate_up, float* out, uint32_t rows, uint32_t f, float limit, float alpha) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * f) return;
    const size_t r = idx / f, c = idx % f;
    const float g = fminf(gate_up[r * 2 * f + c], limit);
    const float u = fminf(fmaxf(gate_up[r * 2 * f + f + c], -limit), limit);
    out[idx] = g * (1.0f / (1.0f + expf(-alpha * g))) * (u + 1.0f);
}

__global__ void unary_f32_kernel(const float* in, uint32_t in_stride, float* out, uint32_t out_stride, uint32_t rows, uint32_t n, uint32_t op) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * n) return;
    const size_t r = idx / n, c = idx % n;
    const float v = in[r * in_stride + c];
    out[r * out_stride + c] = op == 0 ? tanhf(v) : v;
}

__global__ void residual_add_kernel(float* x, const float* a, const float* b, uint32_t length) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= length) return;
    float s = a[idx];
    if (b) s += b[idx];
    x[idx] += s;
}

__global__ void logit_cap_f32_kernel(float* logits, __nv_bfloat16* copy, uint32_t length, float cap, uint32_t has_cap) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= length) return;
    float v = logits[idx];
    if (has_cap) {
        v = cap * tanhf(v / cap);
        logits[idx] = v;
    }
    if (copy) copy[idx] = __float2bfloat16_rn(v);
}

// One CTA. Counting sort of the (row, slot) pairs by expert; pairs of one expert keep token order, so the lists do not depend on the
// thread schedule. rows * top <= 1024 * top pairs; experts <= 1024.
__global__ void __launch_bounds__(1024) table_route_kernel(const uzu_table_route_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ uint32_t counts[];   // [experts + 1]
    const uint32_t* tokens = reinterpret_cast<const uint32_t*>(a.token_ids);
    const int32_t* table = reinterpret_cast<const int32_t*>(a.table);
    uint32_t* offsets = reinterpret_cast<uint32_t*>(a.group_offsets);
    uint32_t* rows_map = reinterpret_cast<uint32_t*>(a.rows_map);
    uint32_t* pair_pos = reinterpret_cast<uint32_t*>(a.pair_pos);
    const uint32_t pairs = a.rows * a.top;
    uint16_t* pe = reinterpret_cast<uint16_t*>(counts + a.experts + 1);   // expert of every pair, staged once
    for (uint32_t e = threadIdx.x; e <= a.experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    auto expert_of = [&](uint32_t p) -> uint32_t {
        const uint32_t tok = tokens[p / a.top];
        const int32_t e = tok < a.vocab ? table[(size_t)tok * a.top + p % a.top] : 0;
        return (e >= 0 && (uint32_t)e < a.experts) ? (uint32_t)e : 0u;
    };
    for (uint32_t p = threadIdx.x; p < pairs; p += blockDim.x) {
        const uint32_t e = expert_of(p);
        pe[p] = (uint16_t)e;
        atomicAdd(&counts[e + 1], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t e = 0; e < a.experts; ++e) counts[e + 1] += counts[e];
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e <= a.experts; e += blockDim.x) offsets[e] = counts[e];
    // stable placement: thread e walks the pairs in order and places those of expert e
    for (uint32_t e = threadIdx.x; e < a.experts; e += blockDim.x) {
        uint32_t at = counts[e];
        if (counts[e + 1] == at) continue;
        for (uint32_t p = 0; p < pairs; ++p) {
            if (pe[p] == e) {
                rows_map[at] = p / a.top;
                pair_pos[p] = at;
                ++at;
            }
        }
    }
}

__global__ void routed_combine_kernel(const float* pairs, const uint32_t* pair_pos, float* out, uint32_t rows, uint32_t top, uint32_t n,
                                      float weight, uint32_t accumulate) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)rows * n) return;
    const size_t r = idx / n, c = idx % n;
    float s = 0.0f;
    for (uint32_t k = 0; k < top; ++k) s += pairs[(size_t)pair_pos[r * top + k] * n + c];
    s *= weight;
    out[idx] = accumulate ? out[idx] + s : s;
}

static inline unsigned blocks256(size_t n) { return (unsigned)((n + 255) / 256); }

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_group_rms_norm_encode(uzu_command_buffer* cmd, const uzu_group_rms_norm_args* a) {
    if (!encodable(cmd, "group_rms_norm")) return;
    if (!a->input || !a->output || a->groups == 0 || a->n % a->groups != 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "group_rms_norm: null operand or the row is not divisible into the groups");
        return;
    }
    if (a->rows == 0 || a->n == 0) return;
    uzu_group_rms_norm_args b = *a;
    if (!b.in_stride) b.in_stride = b.n;
    if (!b.out_stride) b.out_stride = b.n;
    launch(cmd, "group_rms_norm_kernel", group_rms_norm_kernel, dim3(b.rows, b.groups), dim3(256), 0, b);
}

void uzu_embedding_f32_encode(uzu_command_buffer* cmd, uint64_t token_ids, uint64_t table, uint32_t weights_dt, uint64_t output, uint32_t rows,
                              uint32_t vocab, uint32_t n) {
    if (!encodable(cmd, "embedding_f32") || rows == 0 || n == 0) return;
    dim3 grid(blocks256(n), rows);
    if (weights_dt == UZU_DT_BF16)
        launch(cmd, "embedding_f32_kernel", embedding_f32_kernel<__nv_bfloat16>, grid, dim3(256), 0, (const uint32_t*)token_ids, (const __nv_bfloat16*)table, (float*)output, vocab, n);
    else
        launch(cmd, "embedding_f32_kernel", embedding_f32_kernel<float>, grid, dim3(256), 0, (const uint32_t*)token_ids, (const float*)table, (float*)output, vocab, n);
}

void uzu_clamped_glu_encode(uzu_command_buffer* cmd, uint64_t gate_up, uint64_t output, uint32_t rows, uint32_t f, float limit, float alpha) {
    if (!encodable(cmd, "clamped_glu") || rows == 0 || f == 0) return;
    launch(cmd, "clamped_glu_kernel", clamped_glu_kernel, dim3(blocks256((size_t)rows * f)), dim3(256), 0, (const float*)gate_up, (float*)output, rows, f, limit, alpha);
}

void uzu_unary_f32_encode(uzu_command_buffer* cmd, uint64_t input, uint32_t in_stride, uint64_t output, uint32_t out_stride, uint32_t rows,
                          uint32_t n, uint32_t op) {
    if (!encodable(cmd, "unary_f32") || rows == 0 || n == 0) return;
    launch(cmd, "unary_f32_kernel", unary_f32_kernel, dim3(blocks256((size_t)rows * n)), dim3(256), 0, (const float*)input, in_stride, (float*)output, out_stride, rows, n, op);
}

void uzu_residual_add_encode(uzu_command_buffer* cmd, uint64_t x, uint64_t a, uint64_t b, uint32_t length) {
    if (!encodable(cmd, "residual_add") || length == 0) return;
    launch(cmd, "residual_add_kernel", residual_add_kernel, dim3(blocks256(length)), dim3(256), 0, (float*)x, (const float*)a, (const float*)b, length);
}

void uzu_logit_cap_f32_encode(uzu_command_buffer* cmd, uint64_t logits_f32, uint64_t logits_bf16, uint32_t length, float cap, uint32_t has_cap) {
    if (!encodable(cmd, "logit_cap_f32") || length == 0) return;
    launch(cmd, "logit_cap_f32_kernel", logit_cap_f32_kernel, dim3(blocks256(length)), dim3(256), 0, (float*)logits_f32, (__nv_bfloat16*)logits_bf16, length, cap, has_cap);
}

void uzu_table_route_encode(uzu_command_buffer* cmd, const uzu_table_route_args* a) {
    if (!encodable(cmd, "table_route")) return;
    if (!a->token_ids || !a->table || !a->group_offsets || !a->rows_map || !a->pair_pos || a->top == 0 || a->experts == 0 || a->experts > 8192) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "table_route: null operand or bad expert count");
        return;
    }
    if (a->rows == 0) return;
    const size_t smem = (a->experts + 1) * sizeof(uint32_t) + (size_t)a->rows * a->top * sizeof(uint16_t);
    if (smem > 48 * 1024) {
        cmd->record_error(UZU_ERROR_UNSUPPORTED, "table_route: rows * top too large for one pass");
        return;
    }
    launch(cmd, "table_route_kernel", table_route_kernel, dim3(1), dim3(1024), smem, *a);
}

void uzu_routed_combine_encode(uzu_command_buffer* cmd, uint64_t pairs, uint64_t pair_pos, uint64_t output, uint32_t rows, uint32_t top, uint32_t n,
                               float weight, uint32_t accumulate) {
    if (!encodable(cmd, "routed_combine") || rows == 0 || n == 0) return;
    launch(cmd, "routed_combine_kernel", routed_combine_kernel, dim3(blocks256((size_t)rows * n)), dim3(256), 0, (const float*)pairs, (const uint32_t*)pair_pos,
           (float*)output, rows, top, n, weight, accumulate);
}

}  // extern "C"
