// Sigmoid attention: every visible key gets the weight sigmoid(score) on its own -- no softmax, no normalisation over keys, no rotation.
// Positions enter through a per-head distance bias r1 * ln(1 + r2 * (i - j)) taken off the score and through a query temperature
// 1 + coef * ln(floor((p + 1) / every) + 1); a per-head bias is added to the score. Keys and queries are RMS-normed over the whole
// projection (all heads at once) before they are split into heads. Grouped key / value heads; key and value sizes may differ.
//   prepare: per token the normed, temperature-scaled query row (f32) and, for a layer that owns its cache, the normed key row and the
//            value row at the token's position (a layer that reads another layer's cache writes nothing);
//   attend:  one CTA per (query token, head, split of the keys): a warp per key, lanes across the head's channels (coalesced rows),
//            four keys of a warp in flight; because the weights are not normalised the partial results of the splits simply add: the
//            last split to finish (a ticket per query and head) adds them in split order, so no second launch and no dependence on
//            the order of arrival;
//   attend, tensor pipe (sigmoid_attention_mma_kernel): bf16 caches and passes of >= 16 rows.
// The cache holds bf16 or f32 rows; scores, weights and sums are f32.
#include "common.cuh"

namespace uzu {

namespace {

template <typename T>
__device__ __forceinline__ void sa_store(T* p, float v);
template <>
__device__ __forceinline__ void sa_store<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void sa_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// a 4-byte word of a cache row: EPW = 1 element (f32, or one bf16 of an odd-sized row) or 2 bf16 elements
template <typename T, int EPW>
__device__ __forceinline__ void sa_load(const T* p, float (&x)[EPW]) {
    if constexpr (sizeof(T) == 4) {
        x[0] = *p;
    } else if constexpr (EPW == 1) {
        x[0] = __bfloat162float(*p);
    } else {
        const uint32_t u = *reinterpret_cast<const uint32_t*>(p);
        x[0] = __uint_as_float(u << 16);
        x[1] = __uint_as_float(u & 0xffff0000u);
    }
}

__device__ __forceinline__ float sa_temperature(uint32_t pos, uint32_t every, float coef) {
    return every ? 1.0f + coef * logf((float)((pos + 1) / every + 1)) : 1.0f;
}

}  // namespace

// grid (rows, 3): unit 0 the query row, unit 1 the key row, unit 2 the value row
template <typename T>
__global__ void __launch_bounds__(256) sigmoid_attention_prepare_kernel(const uzu_sigmoid_attention_prepare_args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[32];
    const uint32_t t = blockIdx.x, unit = blockIdx.y;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t pos = prefix + t;
    if (unit == 0) {
        if (!a.q) return;
        const float* src = reinterpret_cast<const float*>(a.q) + (size_t)t * a.q_stride;
        const float* sc = reinterpret_cast<const float*>(a.q_scales);
        float* out = reinterpret_cast<float*>(a.query) + (size_t)t * a.q_n;
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x; i < a.q_n; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.q_n + a.epsilon);
        const float temp = sa_temperature(pos, a.temp_every, a.temp_coef);
        for (uint32_t i = threadIdx.x; i < a.q_n; i += blockDim.x) out[i] = src[i] * inv * (sc ? sc[i] : 1.0f) * temp;
    } else if (unit == 1) {
        if (!a.k) return;
        const float* src = reinterpret_cast<const float*>(a.k) + (size_t)t * a.k_stride;
        const float* sc = reinterpret_cast<const float*>(a.k_scales);
        T* out = reinterpret_cast<T*>(a.keys) + (size_t)pos * a.k_n;
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x; i < a.k_n; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.k_n + a.epsilon);
        for (uint32_t i = threadIdx.x; i < a.k_n; i += blockDim.x) sa_store<T>(out + i, src[i] * inv * (sc ? sc[i] : 1.0f));
    } else {
        if (!a.v) return;
        const float* src = reinterpret_cast<const float*>(a.v) + (size_t)t * a.v_stride;
        T* out = reinterpret_cast<T*>(a.values) + (size_t)pos * a.v_n;
        for (uint32_t i = threadIdx.x; i < a.v_n; i += blockDim.x) sa_store<T>(out + i, src[i]);
    }
}

constexpr int SA_WARPS = 4, SA_TILE = 32, SA_UNROLL = 4;

// WPL = words of a head's key / value row per lane (the larger of the two)
template <typename T, int EPW, int WPL>
__global__ void __launch_bounds__(SA_WARPS * 32) sigmoid_attention_kernel(const uzu_sigmoid_attention_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sa_part[];          // [SA_WARPS][vdim]
    __shared__ uint32_t is_last;
    const uint32_t t = blockIdx.x, h = blockIdx.y, split = blockIdx.z, splits = gridDim.z;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t p = prefix + t, keys = p + 1;                 // causal: positions 0 .. own
    const uint32_t tiles = (keys + SA_TILE - 1) / SA_TILE, per = (tiles + splits - 1) / splits;
    const uint32_t j_begin = min(keys, split * per * SA_TILE), j_end = min(keys, (split + 1) * per * SA_TILE);
    const uint32_t g = h / (a.heads / a.kv_heads);
    const uint32_t dwords = (a.dim + EPW - 1) / EPW, vwords = (a.vdim + EPW - 1) / EPW;
    const float r1 = a.dist_r1 ? reinterpret_cast<const float*>(a.dist_r1)[h] : 0.0f;
    const float r2 = a.dist_r2 ? reinterpret_cast<const float*>(a.dist_r2)[h] : 0.0f;
    const float pb = a.head_bias ? reinterpret_cast<const float*>(a.head_bias)[h] : 0.0f;
    float q[WPL][EPW], acc[WPL][EPW];
    {
        const float* qrow = reinterpret_cast<const float*>(a.query) + ((size_t)t * a.heads + h) * a.dim;
#pragma unroll
        for (int i = 0; i < WPL; ++i) {
            const uint32_t w = lane + 32u * i;
#pragma unroll
            for (int e = 0; e < EPW; ++e) {
                q[i][e] = (w < dwords && w * EPW + e < a.dim) ? qrow[w * EPW + e] * a.scale : 0.0f;
                acc[i][e] = 0.0f;
            }
        }
    }
    const T* kbase = reinterpret_cast<const T*>(a.keys) + (size_t)g * a.dim;
    const T* vbase = reinterpret_cast<const T*>(a.values) + (size_t)g * a.vdim;
    const size_t kstride = (size_t)a.kv_heads * a.dim, vstride = (size_t)a.kv_heads * a.vdim;
    for (uint32_t j0 = j_begin + warp * SA_UNROLL; j0 < j_end; j0 += SA_WARPS * SA_UNROLL) {
        float s[SA_UNROLL];
#pragma unroll
        for (int u = 0; u < SA_UNROLL; ++u) {
            const uint32_t j = j0 + u;
            s[u] = 0.0f;
            if (j < j_end) {
                const T* krow = kbase + j * kstride;
#pragma unroll
                for (int i = 0; i < WPL; ++i) {
                    const uint32_t w = lane + 32u * i;
                    if (w < dwords) {
                        float x[EPW];
                        sa_load<T, EPW>(krow + (size_t)w * EPW, x);
#pragma unroll
                        for (int e = 0; e < EPW; ++e) s[u] = fmaf(q[i][e], x[e], s[u]);
                    }
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < SA_UNROLL; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
#pragma unroll
        for (int u = 0; u < SA_UNROLL; ++u) {
            const uint32_t j = j0 + u;
            if (j < j_end) {
                const float score = s[u] - r1 * log1pf(r2 * (float)(p - j)) + pb;
                const float wgt = 1.0f / (1.0f + expf(-score));
                const T* vrow = vbase + j * vstride;
#pragma unroll
                for (int i = 0; i < WPL; ++i) {
                    const uint32_t w = lane + 32u * i;
                    if (w < vwords) {
                        float x[EPW];
                        sa_load<T, EPW>(vrow + (size_t)w * EPW, x);
#pragma unroll
                        for (int e = 0; e < EPW; ++e) acc[i][e] = fmaf(wgt, x[e], acc[i][e]);
                    }
                }
            }
        }
    }
    // the warps' sums meet in warp order
#pragma unroll
    for (int i = 0; i < WPL; ++i) {
        const uint32_t w = lane + 32u * i;
#pragma unroll
        for (int e = 0; e < EPW; ++e)
            if (w < vwords && w * EPW + e < a.vdim) sa_part[warp * a.vdim + w * EPW + e] = acc[i][e];
    }
    __syncthreads();
    float* out = reinterpret_cast<float*>(a.out) + ((size_t)t * a.heads + h) * a.vdim;
    float* mine = splits > 1 ? reinterpret_cast<float*>(a.partials) + (((size_t)t * a.heads + h) * splits + split) * a.vdim : out;
    for (uint32_t c = tid; c < a.vdim; c += blockDim.x) {
        float v = 0.0f;
#pragma unroll
        for (int wq = 0; wq < SA_WARPS; ++wq) v += sa_part[wq * a.vdim + c];
        mine[c] = v;
    }
    if (splits == 1) return;
    __threadfence();
    __syncthreads();
    uint32_t* ticket = reinterpret_cast<uint32_t*>(a.tickets) + (size_t)t * a.heads + h;
    if (tid == 0) is_last = atomicAdd(ticket, 1u) == splits - 1 ? 1u : 0u;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float* parts = reinterpret_cast<const float*>(a.partials) + ((size_t)t * a.heads + h) * splits * a.vdim;
    for (uint32_t c = tid; c < a.vdim; c += blockDim.x) {
        float v = 0.0f;
        for (uint32_t sp = 0; sp < splits; ++sp) v += __ldcg(parts + (size_t)sp * a.vdim + c);
        out[c] = v;
    }
    if (tid == 0) *ticket = 0;
}

template <typename T, int EPW>
static void launch_sigmoid_attention(uzu_command_buffer* cmd, const uzu_sigmoid_attention_args& a, uint32_t splits) {
    const uint32_t words = (std::max(a.dim, a.vdim) + EPW - 1) / EPW, wpl = (words + 31) / 32;
    const dim3 grid(a.rows, a.heads, splits), block(SA_WARPS * 32);
    const size_t smem = (size_t)SA_WARPS * a.vdim * sizeof(float);
    if (wpl <= 1) launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 1>, grid, block, smem, a);
    else if (wpl <= 2) launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 2>, grid, block, smem, a);
    else if (wpl <= 4) launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 4>, grid, block, smem, a);
    else if (wpl <= 8) launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 8>, grid, block, smem, a);
    else launch(cmd, "sigmoid_attention_kernel", sigmoid_attention_kernel<T, EPW, 16>, grid, block, smem, a);
}

bool encode_sigmoid_attention_mma(uzu_command_buffer* cmd, const uzu_sigmoid_attention_args& a);

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_sigmoid_attention_prepare_encode(uzu_command_buffer* cmd, const uzu_sigmoid_attention_prepare_args* a) {
    if (!encodable(cmd, "sigmoid_attention_prepare")) return;
    if ((a->cache_dt != UZU_DT_BF16 && a->cache_dt != UZU_DT_F32) || (a->q && !a->query) || (a->k && !a->keys) || (a->v && !a->values)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "sigmoid_attention_prepare: bad cache type or a projection without its destination");
        return;
    }
    if (a->rows == 0) return;
    if (a->cache_dt == UZU_DT_BF16)
        launch(cmd, "sigmoid_attention_prepare_kernel", sigmoid_attention_prepare_kernel<__nv_bfloat16>, dim3(a->rows, 3), dim3(256), 0, *a);
    else
        launch(cmd, "sigmoid_attention_prepare_kernel", sigmoid_attention_prepare_kernel<float>, dim3(a->rows, 3), dim3(256), 0, *a);
}

void uzu_sigmoid_attention_encode(uzu_command_buffer* cmd, const uzu_sigmoid_attention_args* args) {
    if (!encodable(cmd, "sigmoid_attention")) return;
    uzu_sigmoid_attention_args a = *args;
    if (!a.query || !a.keys || !a.values || !a.out || (a.cache_dt != UZU_DT_BF16 && a.cache_dt != UZU_DT_F32) || a.heads == 0 || a.kv_heads == 0 ||
        a.heads % a.kv_heads != 0 || a.dim == 0 || a.vdim == 0 || a.dim > 512 || a.vdim > 512) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "sigmoid_attention: null operand, bad cache type, head counts that do not divide, or a head size outside 1..512");
        return;
    }
    if (a.rows == 0) return;
    uint32_t splits = std::max(1u, a.splits);
    if (splits > 1 && (!a.partials || !a.tickets)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "sigmoid_attention: key splits need the partial-sum and ticket scratch");
        return;
    }
    if (splits == 1 && encode_sigmoid_attention_mma(cmd, a)) return;
    if (a.cache_dt == UZU_DT_F32) {
        launch_sigmoid_attention<float, 1>(cmd, a, splits);
    } else if (a.dim % 2 == 0 && a.vdim % 2 == 0 && (a.keys & 3) == 0 && (a.values & 3) == 0) {
        launch_sigmoid_attention<__nv_bfloat16, 2>(cmd, a, splits);
    } else {
        launch_sigmoid_attention<__nv_bfloat16, 1>(cmd, a, splits);
    }
}

}  // extern "C"

namespace uzu {
// the tensor-pipe form is added below this line
bool encode_sigmoid_attention_mma(uzu_command_buffer*, const uzu_sigmoid_attention_args&) { return false; }
}  // namespace uzu
