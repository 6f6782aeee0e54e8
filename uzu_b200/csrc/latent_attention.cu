// Latent attention: every head scores against ONE cached row per token, [normed latent c (rank) | rotated shared key part (rot_dim)],
// and sums the latent part of the rows; the per-head key / value up-projections are folded into the query (absorbed key projection)
// and applied after the weighted sum (value projection), both as z-batched dense linears outside these kernels.
//   prepare: per token the cache row (RMS norm of the latent, interleaved-pair rotation of the shared key part) and the rotated part of
//            every head's query;
//   attend:  one CTA per (query token, group of 8 heads): a tile of 32 cache rows is staged once in shared memory as f32 and used by
//            all heads of the group (warp = head, lane = key for the scores, lane = latent channel for the weighted sum); running
//            maximum / normaliser / accumulator in f32 registers (online softmax), causal bound = the query's own position.
// The cache holds bf16 or f32 rows; scores, weights and sums are f32.
#include "common.cuh"

namespace uzu {

template <typename T>
__device__ __forceinline__ void cache_store(T* p, float v);
template <>
__device__ __forceinline__ void cache_store<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void cache_store<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float cache_load(const float* p) { return *p; }
__device__ __forceinline__ float cache_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const uzu_latent_prepare_args a) {
    __shared__ float red[32];
    const uint32_t t = blockIdx.x;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t pos = prefix + t;
    const uint32_t width = a.rank + a.rot_dim;
    const float* cosr = reinterpret_cast<const float*>(a.cosines) + (size_t)pos * a.rot_pairs;
    const float* sinr = reinterpret_cast<const float*>(a.sines) + (size_t)pos * a.rot_pairs;
    if (a.kv) {
        const float* kv = reinterpret_cast<const float*>(a.kv) + (size_t)t * a.kv_stride;
        T* row = reinterpret_cast<T*>(a.cache) + (size_t)pos * width;
        const float* sc = reinterpret_cast<const float*>(a.latent_scales);
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x; i < a.rank; i += blockDim.x) ss = fmaf(kv[i], kv[i], ss);
        ss = block_sum(ss, red);
        const float inv = 1.0f / sqrtf(ss / (float)a.rank + a.epsilon);
        for (uint32_t i = threadIdx.x; i < a.rank; i += blockDim.x) cache_store<T>(row + i, kv[i] * inv * (sc ? sc[i] : 1.0f));
        for (uint32_t i = threadIdx.x; i < a.rot_pairs; i += blockDim.x) {
            const float x0 = kv[a.rank + 2 * i], x1 = kv[a.rank + 2 * i + 1], c = cosr[i], s = sinr[i];
            cache_store<T>(row + a.rank + 2 * i, x0 * c - x1 * s);
            cache_store<T>(row + a.rank + 2 * i + 1, x1 * c + x0 * s);
        }
        for (uint32_t i = 2 * a.rot_pairs + threadIdx.x; i < a.rot_dim; i += blockDim.x) cache_store<T>(row + a.rank + i, kv[a.rank + i]);
    }
    if (a.q) {
        const float* q = reinterpret_cast<const float*>(a.q) + (size_t)t * a.q_stride;
        float* out = reinterpret_cast<float*>(a.query) + (size_t)t * a.heads * width;
        const uint32_t per_head = a.rot_dim;
        for (uint32_t idx = threadIdx.x; idx < a.heads * per_head; idx += blockDim.x) {
            const uint32_t h = idx / per_head, j = idx % per_head;
            const float* src = q + (size_t)h * (a.dim + a.rot_dim) + a.dim;
            float v;
            if (j < 2 * a.rot_pairs) {
                const uint32_t i = j >> 1;
                const float x0 = src[2 * i], x1 = src[2 * i + 1], c = cosr[i], s = sinr[i];
                v = (j & 1) ? x1 * c + x0 * s : x0 * c - x1 * s;
            } else {
                v = src[j];
            }
            out[(size_t)h * width + a.rank + j] = v;
        }
    }
}

constexpr int LA_HEADS = 8, LA_KEYS = 32;

template <typename T, int RV>
__global__ void __launch_bounds__(LA_HEADS * 32) latent_attention_kernel(const uzu_latent_attention_args a) {
    extern __shared__ float la_smem[];
    const uint32_t t = blockIdx.x, h0 = blockIdx.y * LA_HEADS;
    const uint32_t width = a.rank + a.rot_dim, ld = width + 1;
    float* qs = la_smem;                       // [LA_HEADS][width]
    float* tile = qs + LA_HEADS * width;       // [LA_KEYS][ld]
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t prefix = a.dynamic_position ? *reinterpret_cast<const uint32_t*>(a.dynamic_position) : a.prefix;
    const uint32_t keys = prefix + t + 1;      // causal: positions 0 .. own
    const uint32_t head = h0 + warp;
    const bool head_ok = head < a.heads;
    const float* q = reinterpret_cast<const float*>(a.query) + ((size_t)t * a.heads + h0) * width;
    const uint32_t group_heads = min((uint32_t)LA_HEADS, a.heads - h0);
    for (uint32_t i = tid; i < group_heads * width; i += blockDim.x) qs[i] = q[i];
    const T* cache = reinterpret_cast<const T*>(a.cache);
    float m = -INFINITY, l = 0.0f, acc[RV];
#pragma unroll
    for (int i = 0; i < RV; ++i) acc[i] = 0.0f;
    const float* myq = qs + warp * width;
    for (uint32_t j0 = 0; j0 < keys; j0 += LA_KEYS) {
        const uint32_t n = min((uint32_t)LA_KEYS, keys - j0);
        __syncthreads();   // the previous tile is consumed (and, the first time, the queries are staged)
        for (uint32_t i = tid; i < n * width; i += blockDim.x) {
            const uint32_t r = i / width, c = i % width;
            tile[r * ld + c] = cache_load(cache + (size_t)(j0 + r) * width + c);
        }
        __syncthreads();
        if (!head_ok) continue;
        float s = -INFINITY;
        if (lane < n) {
            const float* kr = tile + lane * ld;
            float d0 = 0.0f, d1 = 0.0f;
            uint32_t c = 0;
            for (; c + 1 < width; c += 2) {
                d0 = fmaf(myq[c], kr[c], d0);
                d1 = fmaf(myq[c + 1], kr[c + 1], d1);
            }
            if (c < width) d0 = fmaf(myq[c], kr[c], d0);
            s = (d0 + d1) * a.scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = lane < n ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < RV; ++i) acc[i] *= corr;
        for (uint32_t k = 0; k < n; ++k) {
            const float pk = __shfl_sync(0xffffffffu, p, k);
            const float* vr = tile + k * ld;
#pragma unroll
            for (int i = 0; i < RV; ++i) {
                const uint32_t c = lane + 32 * i;
                if (c < a.rank) acc[i] = fmaf(pk, vr[c], acc[i]);
            }
        }
    }
    if (!head_ok) return;
    float* out = reinterpret_cast<float*>(a.out) + ((size_t)t * a.heads + head) * a.rank;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < RV; ++i) {
        const uint32_t c = lane + 32 * i;
        if (c < a.rank) out[c] = acc[i] * inv;
    }
}

template <typename T, int RV>
static void launch_latent_attention(uzu_command_buffer* cmd, const uzu_latent_attention_args& a) {
    const uint32_t width = a.rank + a.rot_dim;
    const size_t smem = ((size_t)LA_HEADS * width + (size_t)LA_KEYS * (width + 1)) * sizeof(float);
    static std::atomic<uint64_t> done{0};
    if (smem > 48 * 1024) opt_in_dynamic_smem(cmd, latent_attention_kernel<T, RV>, (int)smem, done);
    dim3 grid(a.rows, (a.heads + LA_HEADS - 1) / LA_HEADS);
    latent_attention_kernel<T, RV><<<grid, LA_HEADS * 32, smem, cmd->ctx->stream>>>(a);
    after_launch(cmd, "latent_attention_kernel");
}

template <typename T>
static void dispatch_latent_attention(uzu_command_buffer* cmd, const uzu_latent_attention_args& a) {
    const uint32_t rv = (a.rank + 31) / 32;
    if (rv <= 2) launch_latent_attention<T, 2>(cmd, a);
    else if (rv <= 4) launch_latent_attention<T, 4>(cmd, a);
    else if (rv <= 8) launch_latent_attention<T, 8>(cmd, a);
    else launch_latent_attention<T, 16>(cmd, a);
}

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_latent_prepare_encode(uzu_command_buffer* cmd, const uzu_latent_prepare_args* a) {
    if (!encodable(cmd, "latent_prepare")) return;
    if ((!a->kv && !a->q) || (a->kv && !a->cache) || (a->q && !a->query) || (a->rot_pairs && (!a->cosines || !a->sines)) || 2 * a->rot_pairs > a->rot_dim ||
        (a->cache_dt != UZU_DT_BF16 && a->cache_dt != UZU_DT_F32)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "latent_prepare: inconsistent arguments");
        return;
    }
    if (a->rows == 0) return;
    if (a->cache_dt == UZU_DT_BF16) latent_prepare_kernel<__nv_bfloat16><<<a->rows, 128, 0, cmd->ctx->stream>>>(*a);
    else latent_prepare_kernel<float><<<a->rows, 128, 0, cmd->ctx->stream>>>(*a);
    after_launch(cmd, "latent_prepare_kernel");
}

void uzu_latent_attention_encode(uzu_command_buffer* cmd, const uzu_latent_attention_args* a) {
    if (!encodable(cmd, "latent_attention")) return;
    if (!a->query || !a->cache || !a->out || a->heads == 0 || a->rank == 0 || a->rank > 512 || (a->cache_dt != UZU_DT_BF16 && a->cache_dt != UZU_DT_F32)) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "latent_attention: null operand, or latent size outside 1..512");
        return;
    }
    if ((size_t)(LA_HEADS * (a->rank + a->rot_dim) + LA_KEYS * (a->rank + a->rot_dim + 1)) * 4 > 200 * 1024) {
        cmd->record_error(UZU_ERROR_UNSUPPORTED, "latent_attention: cache row too wide for the shared-memory tile");
        return;
    }
    if (a->rows == 0) return;
    if (a->cache_dt == UZU_DT_BF16) dispatch_latent_attention<__nv_bfloat16>(cmd, *a);
    else dispatch_latent_attention<float>(cmd, *a);
}

}  // extern "C"
