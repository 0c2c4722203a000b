// Routing of a mixture of experts in which every row uses k experts.
//
//   router_topk   z = h Wr^T (float32), s = sigmoid(z); the k experts with the largest s + correction (the lowest
//                 index among equals) are chosen; each weight is scale * s (without the correction), divided by the
//                 sum of the chosen s first when `renormalize`.  A row's logits are one fixed sequence of additions
//                 whatever else the step holds.  `bias` [E] (optional) is added to the logits.  `scoring` = 1
//                 (softmax over the chosen): the k experts with the largest logits z are chosen and their weights are
//                 scale * exp(z_i - max) / sum over the chosen of exp(z_j - max): the other experts' logits do not
//                 enter.
//   pair_tokens   after the (row, choice) pairs have been sorted by expert: the row each sorted pair belongs to.
//   combine       out[t] = add[t] + sum over the row's k pairs of y[pair], in the order of the choices.
//
// The reference routes on the host, one row at a time (src/SharpInference.Engine/ForwardPass.cs:2021-2098); here
// routing stays on the device so that a step's rows can be sorted by expert for grouped products.
#include "common.cuh"

constexpr int TOPK_WARPS = 8;
constexpr int TOPK_MANY_ROWS = 512;   // steps of more rows than this put four rows in a CTA (a router row is fetched
                                      // once for all of them); smaller steps one, for more CTAs

// One CTA per TOPK_ROWS rows (1 or 4): warp w forms the logits of experts w, w + 8, ... for each of the CTA's rows (a lane
// adds its elements of a row in ascending order in four interleaved chains, the chains and then the lanes are added
// in a fixed order: a row's logits do not depend on its neighbours), then warp r picks the k best of row r.
template <int TOPK_ROWS>
__global__ void __launch_bounds__(TOPK_WARPS * 32)
router_topk_kernel(const float* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ correction,
                   int T, int H, int E, int k, float scale, int renormalize, int* __restrict__ expert_id,
                   float* __restrict__ weight, float* __restrict__ scores_out, int stage_rows,
                   const float* __restrict__ bias, int scoring) {
    extern __shared__ float smem[];                       // per row s [E], choice [E]; then the rows [ROWS][H] if they fit
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * TOPK_ROWS;
    const int rows = min(TOPK_ROWS, T - t0);
    const float* row[TOPK_ROWS];
#pragma unroll
    for (int r = 0; r < TOPK_ROWS; ++r) row[r] = h + (size_t)(t0 + min(r, rows - 1)) * H;
    if (stage_rows) {                                     // the rows are read from memory once, by all warps together
        float* rows_s = smem + (size_t)TOPK_ROWS * 2 * E;
        for (int i = threadIdx.x; i < rows * H; i += TOPK_WARPS * 32) rows_s[i] = h[(size_t)t0 * H + i];
        __syncthreads();
#pragma unroll
        for (int r = 0; r < TOPK_ROWS; ++r) row[r] = rows_s + (size_t)min(r, rows - 1) * H;
    }
    for (int e = warp; e < E; e += TOPK_WARPS) {
        const float* w = wr + (size_t)e * H;
        float acc[TOPK_ROWS][4];
#pragma unroll
        for (int r = 0; r < TOPK_ROWS; ++r)
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[r][u] = 0.0f;
        int i = lane;
        for (; i + 96 < H; i += 128) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float wv = w[i + 32 * u];
#pragma unroll
                for (int r = 0; r < TOPK_ROWS; ++r) acc[r][u] = fmaf(row[r][i + 32 * u], wv, acc[r][u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 3; ++u) {                      // what is left: up to three more elements a lane
            const int ii = i + 32 * u;
            if (ii < H) {
                const float wv = w[ii];
#pragma unroll
                for (int r = 0; r < TOPK_ROWS; ++r) acc[r][u] = fmaf(row[r][ii], wv, acc[r][u]);
            }
        }
#pragma unroll
        for (int r = 0; r < TOPK_ROWS; ++r) {
            const float z = warp_sum((acc[r][0] + acc[r][1]) + (acc[r][2] + acc[r][3])) + (bias ? bias[e] : 0.0f);
            if (lane == 0 && r < rows) {
                const float s = scoring == 1 ? z : 1.0f / (1.0f + expf(-z));
                smem[(size_t)r * 2 * E + e] = s;
                smem[(size_t)r * 2 * E + E + e] = correction ? s + correction[e] : s;
                if (scores_out) scores_out[(size_t)(t0 + r) * E + e] = s;
            }
        }
    }
    __syncthreads();
    if (warp >= rows) return;
    const int t = t0 + warp;
    float* s_s = smem + (size_t)warp * 2 * E;
    float* c_s = s_s + E;
    float total = 0.0f, top = 0.0f;
    int mine = 0;                                          // lane j keeps the j-th choice
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float c = c_s[e];
            if (c > best) { best = c; at = e; }          // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= E) at = j < E ? j : 0;                   // every score was NaN: any expert, but a valid one
        if (lane == 0) {
            expert_id[(size_t)t * k + j] = at;
            c_s[at] = -INFINITY;
        }
        if (lane == j) mine = at;
        if (scoring == 1) {                                // the first choice has the largest logit
            if (j == 0) top = s_s[at];
            total += expf(s_s[at] - top);
        } else {
            total += s_s[at];
        }
        __syncwarp();
    }
    if (scoring == 1) {
        if (lane < k) weight[(size_t)t * k + lane] = expf(s_s[mine] - top) * (scale / total);
        return;
    }
    const float factor = renormalize ? scale / total : scale;
    if (lane < k) weight[(size_t)t * k + lane] = s_s[mine] * factor;      // k <= 32 is checked by the host
}

SHARPI_API int sharpi_router_topk(const float* h, const float* wr, const float* correction, int T, int H, int E, int k,
                                  float scale, int renormalize, int* expert_id, float* weight, float* scores_out,
                                  const float* bias, int scoring, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (H <= 0 || E <= 0 || k <= 0 || k > E || k > 32 || (scoring != 0 && scoring != 1)) return SHARPI_BAD_ARGUMENT;
    const int per_cta = T > TOPK_MANY_ROWS ? 4 : 1;
    size_t smem = (size_t)per_cta * 2 * E * sizeof(float);
    if (smem > 48 * 1024) return SHARPI_BAD_ARGUMENT;
    const int stage_rows = smem + (size_t)per_cta * H * sizeof(float) <= 48 * 1024;
    if (stage_rows) smem += (size_t)per_cta * H * sizeof(float);
    if (per_cta == 4)
        router_topk_kernel<4><<<(T + 3) / 4, TOPK_WARPS * 32, smem, stream>>>(
            h, wr, correction, T, H, E, k, scale, renormalize, expert_id, weight, scores_out, stage_rows, bias, scoring);
    else
        router_topk_kernel<1><<<T, TOPK_WARPS * 32, smem, stream>>>(
            h, wr, correction, T, H, E, k, scale, renormalize, expert_id, weight, scores_out, stage_rows, bias, scoring);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

__global__ void pair_tokens_kernel(const int* __restrict__ sorted_pairs, int P, int k, int* __restrict__ tokens) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < P) tokens[i] = sorted_pairs[i] / k;
}

SHARPI_API int sharpi_moe_pair_tokens(const int* sorted_pairs, int P, int k, int* tokens, cudaStream_t stream) {
    if (P <= 0) return SHARPI_OK;
    if (k <= 0) return SHARPI_BAD_ARGUMENT;
    pair_tokens_kernel<<<(P + 255) / 256, 256, 0, stream>>>(sorted_pairs, P, k, tokens);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const float* add, float* out,      // out may be add
                                   int k, int H) {
    const int t = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x) {
        float acc = add ? add[(size_t)t * H + i] : 0.0f;
        for (int j = 0; j < k; ++j) acc += y[((size_t)t * k + j) * H + i];
        out[(size_t)t * H + i] = acc;
    }
}

__global__ void moe_combine_vec4_kernel(const float4* __restrict__ y, const float4* add, float4* out, int k, int H4) {
    const int t = blockIdx.x;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H4; i += gridDim.y * blockDim.x) {
        float4 acc = add ? add[(size_t)t * H4 + i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int j = 0; j < k; ++j) {
            const float4 v = y[((size_t)t * k + j) * H4 + i];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        out[(size_t)t * H4 + i] = acc;
    }
}

SHARPI_API int sharpi_moe_combine(const float* y, const float* add, float* out, int T, int k, int H,
                                  cudaStream_t stream) {
    if (T <= 0 || H <= 0) return SHARPI_OK;
    if (k <= 0) return SHARPI_BAD_ARGUMENT;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(add) | reinterpret_cast<uintptr_t>(out);
    if (H % 4 == 0 && (ptrs & 15) == 0) {               // same additions in the same order, four columns a thread
        int by4 = (H / 4 + 255) / 256;
        if (by4 > 64) by4 = 64;
        moe_combine_vec4_kernel<<<dim3(T, by4), 256, 0, stream>>>((const float4*)y, (const float4*)add, (float4*)out, k, H / 4);
        SHARPI_CHECK_LAUNCH();
        return SHARPI_OK;
    }
    int by = (H + 255) / 256;
    if (by > 64) by = 64;
    moe_combine_kernel<<<dim3(T, by), 256, 0, stream>>>(y, add, out, k, H);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}
