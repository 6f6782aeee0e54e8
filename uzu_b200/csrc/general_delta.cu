// Generalized delta rule (per head a dim x dim f32 state S, key channel x value channel):
//     S <- diag(d) S - (a * u)(u^T S) + k v^T,   out = S^T r
// with decay d = exp(-e^-1/2 * sigmoid(.)), removal rate a = sigmoid(.), unit key u = k / sqrt(sum k^2 + 1e-6), all formed in f32 here
// from the raw projections. One launch walks the `rows` tokens of a pass in order with the state on chip: the value columns of a head are
// independent (u^T S is a per-column dot product), so the grid is (column blocks of 32, heads) and a CTA keeps its dim x 32 slice of
// the state in registers -- warp p owns key channels [16p, 16p + 16), lane c owns column c. Per token the CTA forms the head's vectors
// once in shared memory, every thread contributes a partial of u^T S and of S^T r, and partials meet in shared memory in warp order
// (a fixed order: one token at a time or a thousand in one launch give the same bits). The next token's inputs are requested
// before the current token is worked on. The same kernel is the decode step (rows = 1). This block-wide form serves head sizes above
// 128 and those that are no multiple of 4; smaller heads take general_delta_warp_kernel below.
#include <cstdlib>

#include "common.cuh"

namespace uzu {

constexpr int GD_PART = 16;   // key channels per warp

__global__ void __launch_bounds__(1024) general_delta_kernel(const uzu_general_delta_args a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float gd_smem[];
    const uint32_t dim = a.dim, head = blockIdx.y;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, parts = blockDim.x >> 5;
    const uint32_t col = blockIdx.x * 32 + lane;
    const bool col_ok = col < dim;
    // shared memory: 2 x { d, au, u, k, r : dim each } + 2 x zpart[parts][32] + 2 x opart[parts][32] + 2 x ssq[32]
    float* vec = gd_smem;                                  // [2][5][dim]
    float* zpart = vec + 2 * 5 * dim;                      // [2][parts][32]
    float* opart = zpart + 2 * parts * 32;                 // [2][parts][32]
    float* ssq = opart + 2 * parts * 32;                   // [2][32]
    const uint32_t i0 = warp * GD_PART;
    const uint32_t cnt = i0 < dim ? min((uint32_t)GD_PART, dim - i0) : 0u;
    float* state = reinterpret_cast<float*>(a.state) + (size_t)head * dim * dim;
    float S[GD_PART];
#pragma unroll
    for (int i = 0; i < GD_PART; ++i) S[i] = ((uint32_t)i < cnt && col_ok) ? state[(size_t)(i0 + i) * dim + col] : 0.0f;

    const float* pr = reinterpret_cast<const float*>(a.r);
    const float* pk = reinterpret_cast<const float*>(a.k);
    const float* pv = reinterpret_cast<const float*>(a.v);
    const float* pa = reinterpret_cast<const float*>(a.rate_logit);
    const float* pd = reinterpret_cast<const float*>(a.decay_logit);
    const uint32_t hc = head * dim;
    const bool prep = tid < dim;
    const float rate_b = (prep && a.rate_bias) ? reinterpret_cast<const float*>(a.rate_bias)[hc + tid] : 0.0f;
    const float decay_b = (prep && a.decay_bias) ? reinterpret_cast<const float*>(a.decay_bias)[hc + tid] : 0.0f;
    float nk = 0.0f, nr = 0.0f, na = 0.0f, nd = 0.0f, nv = 0.0f;
    auto request = [&](uint32_t t) {
        if (prep) {
            nk = pk[(size_t)t * a.k_stride + hc + tid];
            nr = pr[(size_t)t * a.r_stride + hc + tid];
            na = pa[(size_t)t * a.rate_stride + hc + tid];
            nd = pd[(size_t)t * a.decay_stride + hc + tid];
        }
        if (col_ok) nv = pv[(size_t)t * a.v_stride + hc + col];
    };
    request(0);
    for (uint32_t t = 0; t < a.rows; ++t) {
        const uint32_t b = t & 1;
        float* vd = vec + (size_t)b * 5 * dim;
        float *vau = vd + dim, *vu = vau + dim, *vk = vu + dim, *vr = vk + dim;
        const float kk = nk, rr = nr, al = na + rate_b, dl = nd + decay_b, vv = nv;
        if (t + 1 < a.rows) request(t + 1);
        const float sq = warp_sum(prep ? kk * kk : 0.0f);
        if (lane == 0) ssq[b * 32 + warp] = sq;
        __syncthreads();
        if (prep) {
            float total = 0.0f;
            for (uint32_t w = 0; w < parts; ++w) total += ssq[b * 32 + w];
            const float u = kk / sqrtf(total + 1e-6f);
            const float rate = 1.0f / (1.0f + expf(-al));
            const float decay = expf(-0.60653065971263342f * (1.0f / (1.0f + expf(-dl))));
            vd[tid] = decay;
            vau[tid] = rate * u;
            vu[tid] = u;
            vk[tid] = kk;
            vr[tid] = rr;
        }
        __syncthreads();
        float zp = 0.0f;
#pragma unroll
        for (int i = 0; i < GD_PART; ++i)
            if ((uint32_t)i < cnt) zp = fmaf(vu[i0 + i], S[i], zp);
        zpart[(b * parts + warp) * 32 + lane] = zp;
        __syncthreads();
        float z = 0.0f;
        for (uint32_t w = 0; w < parts; ++w) z += zpart[(b * parts + w) * 32 + lane];
        float op = 0.0f;
#pragma unroll
        for (int i = 0; i < GD_PART; ++i) {
            if ((uint32_t)i < cnt) {
                const float s = fmaf(vk[i0 + i], vv, fmaf(-vau[i0 + i], z, vd[i0 + i] * S[i]));
                S[i] = s;
                op = fmaf(s, vr[i0 + i], op);
            }
        }
        opart[(b * parts + warp) * 32 + lane] = op;
        __syncthreads();
        if (warp == 0 && col_ok) {
            float o = 0.0f;
            for (uint32_t w = 0; w < parts; ++w) o += opart[(b * parts + w) * 32 + lane];
            reinterpret_cast<float*>(a.out)[(size_t)t * a.heads * dim + hc + col] = o;
        }
    }
#pragma unroll
    for (int i = 0; i < GD_PART; ++i)
        if ((uint32_t)i < cnt && col_ok) state[(size_t)(i0 + i) * dim + col] = S[i];
}

// Head sizes up to 64 (the 96 / 128 instances exist but spill registers and lose to the block-wide form; they are not selected):
// ONE WARP owns a 32-column slice of a head's state with all key channels in registers (lane = value column,
// S[i] = state[i][column]). u^T S and S^T r are then sums inside a lane, in channel order: no shuffles, no block barriers. Per token the
// warp forms the head's vectors (decay, rate * unit key, unit key, key, receptance) once in shared memory -- the unit key needs one warp
// sum -- and every lane runs its column: z = sum_i u_i S_i;  S_i <- d_i S_i - (a u)_i z + k_i v;  o = sum_i S_i r_i. The next token's raw
// inputs are requested before the current token is worked on.
template <int DMAX>
__global__ void __launch_bounds__(32) general_delta_warp_kernel(const uzu_general_delta_args a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ __align__(16) float vec[5][DMAX];          // d, a*u, u, k, r of the current token
    const uint32_t dim = a.dim, head = blockIdx.y, lane = threadIdx.x;
    const uint32_t col = blockIdx.x * 32 + lane;
    const bool col_ok = col < dim;
    float* state = reinterpret_cast<float*>(a.state) + (size_t)head * dim * dim;
    float S[DMAX];
#pragma unroll
    for (int i = 0; i < DMAX; ++i) S[i] = ((uint32_t)i < dim && col_ok) ? state[(size_t)i * dim + col] : 0.0f;
    const float* pr = reinterpret_cast<const float*>(a.r);
    const float* pk = reinterpret_cast<const float*>(a.k);
    const float* pv = reinterpret_cast<const float*>(a.v);
    const float* pa = reinterpret_cast<const float*>(a.rate_logit);
    const float* pd = reinterpret_cast<const float*>(a.decay_logit);
    const uint32_t hc = head * dim;
    constexpr int PER = DMAX / 32;                         // channels a lane prepares: lane, lane + 32, ...
    float rate_b[PER], decay_b[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const uint32_t c = lane + 32 * j;
        rate_b[j] = (c < dim && a.rate_bias) ? reinterpret_cast<const float*>(a.rate_bias)[hc + c] : 0.0f;
        decay_b[j] = (c < dim && a.decay_bias) ? reinterpret_cast<const float*>(a.decay_bias)[hc + c] : 0.0f;
    }
    float nk[PER], nr[PER], na[PER], nd[PER], nv = 0.0f;
    auto request = [&](uint32_t t) {
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const uint32_t c = lane + 32 * j;
            const bool ok = c < dim;
            nk[j] = ok ? pk[(size_t)t * a.k_stride + hc + c] : 0.0f;
            nr[j] = ok ? pr[(size_t)t * a.r_stride + hc + c] : 0.0f;
            na[j] = ok ? pa[(size_t)t * a.rate_stride + hc + c] : 0.0f;
            nd[j] = ok ? pd[(size_t)t * a.decay_stride + hc + c] : 0.0f;
        }
        nv = col_ok ? pv[(size_t)t * a.v_stride + hc + col] : 0.0f;
    };
    request(0);
    for (uint32_t t = 0; t < a.rows; ++t) {
        float kk[PER], rr[PER], al[PER], dl[PER];
        float sq = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            kk[j] = nk[j]; rr[j] = nr[j]; al[j] = na[j] + rate_b[j]; dl[j] = nd[j] + decay_b[j];
            sq = fmaf(kk[j], kk[j], sq);
        }
        const float vv = nv;
        if (t + 1 < a.rows) request(t + 1);
        const float inv = 1.0f / sqrtf(warp_sum(sq) + 1e-6f);
        __syncwarp();                                      // the previous token's vectors are no longer read
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const uint32_t c = lane + 32 * j;
            if (c < dim) {
                const float u = kk[j] * inv;
                vec[0][c] = expf(-0.60653065971263342f * (1.0f / (1.0f + expf(-dl[j]))));
                vec[1][c] = (1.0f / (1.0f + expf(-al[j]))) * u;
                vec[2][c] = u;
                vec[3][c] = kk[j];
                vec[4][c] = rr[j];
            }
        }
        __syncwarp();
        // four running sums each for u^T S and S^T r: neighbouring channels do not wait for one another's multiply-add
        float z0 = 0.0f, z1 = 0.0f, z2 = 0.0f, z3 = 0.0f;
#pragma unroll
        for (int i = 0; i < DMAX; i += 4) {
            if ((uint32_t)i < dim) {                       // dim is a multiple of 4 on this path
                const float4 u4 = *reinterpret_cast<const float4*>(&vec[2][i]);
                z0 = fmaf(u4.x, S[i], z0);
                z1 = fmaf(u4.y, S[i + 1], z1);
                z2 = fmaf(u4.z, S[i + 2], z2);
                z3 = fmaf(u4.w, S[i + 3], z3);
            }
        }
        const float z = (z0 + z1) + (z2 + z3);
        float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
        for (int i = 0; i < DMAX; i += 4) {
            if ((uint32_t)i < dim) {
                const float4 d4 = *reinterpret_cast<const float4*>(&vec[0][i]);
                const float4 au4 = *reinterpret_cast<const float4*>(&vec[1][i]);
                const float4 k4 = *reinterpret_cast<const float4*>(&vec[3][i]);
                const float4 r4 = *reinterpret_cast<const float4*>(&vec[4][i]);
                S[i] = fmaf(k4.x, vv, fmaf(-au4.x, z, d4.x * S[i]));
                S[i + 1] = fmaf(k4.y, vv, fmaf(-au4.y, z, d4.y * S[i + 1]));
                S[i + 2] = fmaf(k4.z, vv, fmaf(-au4.z, z, d4.z * S[i + 2]));
                S[i + 3] = fmaf(k4.w, vv, fmaf(-au4.w, z, d4.w * S[i + 3]));
                o0 = fmaf(S[i], r4.x, o0);
                o1 = fmaf(S[i + 1], r4.y, o1);
                o2 = fmaf(S[i + 2], r4.z, o2);
                o3 = fmaf(S[i + 3], r4.w, o3);
            }
        }
        const float o = (o0 + o1) + (o2 + o3);
        if (col_ok) reinterpret_cast<float*>(a.out)[(size_t)t * a.heads * dim + hc + col] = o;
    }
#pragma unroll
    for (int i = 0; i < DMAX; ++i)
        if ((uint32_t)i < dim && col_ok) state[(size_t)i * dim + col] = S[i];
}

// one warp per (row, head)
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const uzu_head_norm_gate_args a) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const uint32_t unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= a.rows * a.heads) return;
    const uint32_t row = unit / a.heads, h = unit % a.heads;
    const float* x = reinterpret_cast<const float*>(a.x) + (size_t)row * a.x_stride + (size_t)h * a.dim;
    const float* gate = a.gate ? reinterpret_cast<const float*>(a.gate) + (size_t)row * a.gate_stride + (size_t)h * a.dim : nullptr;
    const float* sc = a.scales ? reinterpret_cast<const float*>(a.scales) + (size_t)h * a.dim : nullptr;
    float* out = reinterpret_cast<float*>(a.out) + (size_t)row * a.out_stride + (size_t)h * a.dim;
    float inv = 1.0f;
    if (a.normalize) {
        float ss = 0.0f;
        for (uint32_t i = lane; i < a.dim; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)a.dim + a.epsilon);
    }
    for (uint32_t i = lane; i < a.dim; i += 32) {
        float v = x[i] * inv;
        if (sc) v *= sc[i];
        if (gate) v *= 1.0f / (1.0f + expf(-gate[i]));
        out[i] = v;
    }
}

}  // namespace uzu

extern "C" {
using namespace uzu;

void uzu_general_delta_encode(uzu_command_buffer* cmd, const uzu_general_delta_args* a) {
    if (!encodable(cmd, "general_delta")) return;
    if (!a->r || !a->k || !a->v || !a->rate_logit || !a->decay_logit || !a->state || !a->out || a->dim == 0 || a->dim > 32 * GD_PART || a->heads == 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "general_delta: null operand or head size outside 1..512");
        return;
    }
    if (a->rows == 0) return;
    static const int warp_max_dim = [] { const char* e = getenv("UZU_DELTA_WARP_MAX_DIM"); return e ? atoi(e) : 64; }();   // A/B runs; measured: 1.6x (dim 48) / 1.3x (dim 64) faster than the block-wide form, slower at 128 (registers spill)
    if (a->dim % 4 == 0 && a->dim <= (uint32_t)warp_max_dim) {          // one warp per (32 value columns, head), the state in registers
        const dim3 grid((a->dim + 31) / 32, a->heads);
        if (a->dim <= 32) launch(cmd, "general_delta_warp_kernel", general_delta_warp_kernel<32>, grid, dim3(32), 0, *a);
        else if (a->dim <= 64) launch(cmd, "general_delta_warp_kernel", general_delta_warp_kernel<64>, grid, dim3(32), 0, *a);
        else if (a->dim <= 96) launch(cmd, "general_delta_warp_kernel", general_delta_warp_kernel<96>, grid, dim3(32), 0, *a);
        else launch(cmd, "general_delta_warp_kernel", general_delta_warp_kernel<128>, grid, dim3(32), 0, *a);
        return;
    }
    const uint32_t parts = (a->dim + GD_PART - 1) / GD_PART;
    const size_t smem = ((size_t)2 * 5 * a->dim + (size_t)4 * parts * 32 + 64) * sizeof(float);
    static std::atomic<uint64_t> done{0};
    if (smem > 48 * 1024) opt_in_dynamic_smem(cmd, general_delta_kernel, (int)smem, done);
    launch(cmd, "general_delta_kernel", general_delta_kernel, dim3((a->dim + 31) / 32, a->heads), dim3(parts * 32), smem, *a);
}

void uzu_head_norm_gate_encode(uzu_command_buffer* cmd, const uzu_head_norm_gate_args* a) {
    if (!encodable(cmd, "head_norm_gate")) return;
    if (!a->x || !a->out || a->dim == 0 || a->heads == 0) {
        cmd->record_error(UZU_ERROR_INVALID_ARGUMENT, "head_norm_gate: null operand");
        return;
    }
    if (a->rows == 0) return;
    uzu_head_norm_gate_args b = *a;
    if (!b.x_stride) b.x_stride = b.heads * b.dim;
    if (!b.gate_stride) b.gate_stride = b.heads * b.dim;
    if (!b.out_stride) b.out_stride = b.heads * b.dim;
    const uint32_t units = b.rows * b.heads;
    launch(cmd, "head_norm_gate_kernel", head_norm_gate_kernel, dim3((units + 3) / 4), dim3(128), 0, b);
}

}  // extern "C"
