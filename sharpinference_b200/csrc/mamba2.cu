// The state-space-duality recurrence (Mamba-2) from per-request state, walked row by row, and the gated norm in
// groups behind it.
//
//   sharpi_ssd_scan     per head h (its group g = h / (heads / groups)), for the rows of a request in order:
//                         dt = softplus(dt_raw[h] + dt_bias[h]);  a = exp(-exp(A_log[h]) * dt)
//                         S[n][v] <- a S[n][v] + dt B_g[n] x_h[v]        (S is N x P per head, float32)
//                         y_h[v]  = sum_n S[n][v] C_g[n] + D[h] x_h[v]
//                       x, B and C are columns of one float32 matrix (the convolution's output), dt_raw columns of
//                       another (the fused input projection).  A block serves one (request, head, 32 value columns);
//                       eight lanes share a column, each keeping N / 8 of its states in registers; the rows of a
//                       chunk of SSD_CH tokens are staged in shared memory together.  The sum over the states is a
//                       fixed order inside a lane and a fixed tree across the eight lanes, and the walk over a
//                       request's rows is sequential, so a row's result does not depend on how a prompt was cut or
//                       batched.  The state is read at the start of a portion and stored behind its last row.
//   sharpi_gated_group_norm   u = y * silu(z);  out = u / sqrt(mean_part(u^2) + eps) * w, the width in `parts` equal
//                       consecutive parts, each with its own mean (float32; output in the activation dtype).
#include "common.cuh"

constexpr int SSD_THREADS = 256;
constexpr int SSD_LANES = 8;                         // lanes that share one value column
constexpr int SSD_COLS = SSD_THREADS / SSD_LANES;    // value columns a block
constexpr int SSD_CH = 16;                           // rows staged together
constexpr int SSD_MAX_STATES = 256;

struct SsdArgs {
    const float* xbc;        // [T, ld_x]: x at col_x (heads * P), B at col_b (groups * N), C at col_c
    int ld_x, col_x, col_b, col_c;
    const float* dt;         // [T, ld_dt]: raw step sizes at col_dt (heads)
    int ld_dt, col_dt;
    const float* dt_bias;    // [heads]
    const float* a_log;      // [heads]
    const float* dskip;      // [heads]
    const int* row_offsets;  // [B + 1]
    const int* state_slots;  // [B]
    float* state;            // [slots][heads][N][P]
    long long state_stride;
    float* y;                // [T, heads * P]
    int heads, groups, N, P;
};

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

template <int NPL>           // states a lane: N <= 8 * NPL
__global__ void __launch_bounds__(SSD_THREADS) ssd_scan_kernel(SsdArgs a) {
    extern __shared__ float smem[];
    const int N = a.N, P = a.P;
    float* b_s = smem;                      // [SSD_CH][N]
    float* c_s = b_s + SSD_CH * N;          // [SSD_CH][N]
    float* x_s = c_s + SSD_CH * N;          // [SSD_CH][SSD_COLS]
    float* dt_s = x_s + SSD_CH * SSD_COLS;  // [SSD_CH] step sizes, then [SSD_CH] decays
    pdl_wait();
    const int req = blockIdx.z, h = blockIdx.y;
    const int g = h / (a.heads / a.groups);
    const int first = a.row_offsets[req], rows = a.row_offsets[req + 1] - first;
    if (rows <= 0) return;
    const int lane = threadIdx.x % SSD_LANES;
    const int col = threadIdx.x / SSD_LANES;
    const int v = blockIdx.x * SSD_COLS + col;
    const bool live = v < P;
    float* st = a.state + (size_t)a.state_slots[req] * a.state_stride + (size_t)h * N * P;
    float S[NPL];
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = lane + SSD_LANES * j;
        S[j] = (live && n < N) ? st[(size_t)n * P + v] : 0.0f;
    }
    const float decay_rate = -expf(a.a_log[h]);
    const float bias = a.dt_bias[h], dsk = a.dskip[h];
    for (int r0 = 0; r0 < rows; r0 += SSD_CH) {
        const int nr = min(SSD_CH, rows - r0);
        __syncthreads();                    // the previous chunk is no longer read
        for (int i = threadIdx.x; i < nr * N; i += SSD_THREADS) {
            const int r = i / N, n = i % N;
            const float* row = a.xbc + (size_t)(first + r0 + r) * a.ld_x;
            b_s[r * N + n] = row[a.col_b + g * N + n];
            c_s[r * N + n] = row[a.col_c + g * N + n];
        }
        for (int i = threadIdx.x; i < nr * SSD_COLS; i += SSD_THREADS) {
            const int r = i / SSD_COLS, c = i % SSD_COLS;
            const int vv = blockIdx.x * SSD_COLS + c;
            x_s[i] = vv < P ? a.xbc[(size_t)(first + r0 + r) * a.ld_x + a.col_x + h * P + vv] : 0.0f;
        }
        if (threadIdx.x < nr) {
            const float d = softplus_f(a.dt[(size_t)(first + r0 + threadIdx.x) * a.ld_dt + a.col_dt + h] + bias);
            dt_s[threadIdx.x] = d;
            dt_s[SSD_CH + threadIdx.x] = expf(decay_rate * d);
        }
        __syncthreads();
        for (int r = 0; r < nr; ++r) {
            const float d = dt_s[r], decay = dt_s[SSD_CH + r];
            const float xv = x_s[r * SSD_COLS + col];
            const float dx = d * xv;
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < NPL; ++j) {
                const int n = lane + SSD_LANES * j;
                if (n < N) {
                    S[j] = decay * S[j] + dx * b_s[r * N + n];
                    acc += S[j] * c_s[r * N + n];
                }
            }
#pragma unroll
            for (int o = SSD_LANES / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0 && live) a.y[(size_t)(first + r0 + r) * a.heads * P + h * P + v] = acc + dsk * xv;
        }
    }
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = lane + SSD_LANES * j;
        if (live && n < N) st[(size_t)n * P + v] = S[j];
    }
}

SHARPI_API int sharpi_ssd_scan(const float* xbc, int ld_x, int col_x, int col_b, int col_c, const float* dt, int ld_dt,
                               int col_dt, const float* dt_bias, const float* a_log, const float* dskip,
                               const int* row_offsets, const int* state_slots, float* state, long long state_stride,
                               float* y, int T, int B, int heads, int groups, int N, int P, cudaStream_t stream) {
    if (T <= 0 || B <= 0) return SHARPI_OK;
    if (heads <= 0 || groups <= 0 || heads % groups != 0 || N <= 0 || N > SSD_MAX_STATES || P <= 0 || heads > 65535 ||
        B > 65535 || col_x + heads * P > ld_x || col_b + groups * N > ld_x || col_c + groups * N > ld_x ||
        col_dt + heads > ld_dt)
        return SHARPI_BAD_ARGUMENT;
    SsdArgs a;
    a.xbc = xbc; a.ld_x = ld_x; a.col_x = col_x; a.col_b = col_b; a.col_c = col_c; a.dt = dt; a.ld_dt = ld_dt;
    a.col_dt = col_dt; a.dt_bias = dt_bias; a.a_log = a_log; a.dskip = dskip; a.row_offsets = row_offsets;
    a.state_slots = state_slots; a.state = state; a.state_stride = state_stride; a.y = y; a.heads = heads;
    a.groups = groups; a.N = N; a.P = P;
    const dim3 grid((P + SSD_COLS - 1) / SSD_COLS, heads, B);
    const size_t smem = (size_t)(2 * SSD_CH * N + SSD_CH * SSD_COLS + 2 * SSD_CH) * sizeof(float);
    const int per_lane = (N + SSD_LANES - 1) / SSD_LANES;
#define SSD_CASE(NPL)                                                                    \
    do {                                                                                 \
        auto kern = ssd_scan_kernel<NPL>;                                                \
        SHARPI_LAUNCH_PDL(kern, grid, SSD_THREADS, smem, stream, a);                     \
    } while (0)
    if (per_lane <= 1) SSD_CASE(1);
    else if (per_lane <= 2) SSD_CASE(2);
    else if (per_lane <= 4) SSD_CASE(4);
    else if (per_lane <= 8) SSD_CASE(8);
    else if (per_lane <= 16) SSD_CASE(16);
    else SSD_CASE(32);
#undef SSD_CASE
    return SHARPI_OK;
}

template <typename TO>
__global__ void __launch_bounds__(256)
gated_group_norm_kernel(const float* y, const float* z, int ld_z, const float* __restrict__ w, float eps, int width,
                        int parts, TO* out) {
    __shared__ float scratch[32];
    pdl_wait();
    const int t = blockIdx.x, part = blockIdx.y;
    const int n = width / parts;
    const float* yr = y + (size_t)t * width + (size_t)part * n;
    const float* zr = z + (size_t)t * ld_z + (size_t)part * n;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n; i += 256) {
        const float g = zr[i];
        const float u = yr[i] * (g / (1.0f + expf(-g)));
        ss += u * u;
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)n + eps);
    TO* orow = out + (size_t)t * width + (size_t)part * n;
    for (int i = threadIdx.x; i < n; i += 256) {
        const float g = zr[i];
        const float u = yr[i] * (g / (1.0f + expf(-g)));
        orow[i] = from_float<TO>(u * scale * w[(size_t)part * n + i]);
    }
}

SHARPI_API int sharpi_gated_group_norm(const float* y, const float* z, int ld_z, const float* w, float eps, int T,
                                       int width, int parts, void* out, int out_dtype, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (width <= 0 || parts <= 0 || width % parts != 0 || parts > 65535 || ld_z < width) return SHARPI_BAD_ARGUMENT;
    const dim3 grid(T, parts);
    if (out_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(gated_group_norm_kernel<float>, grid, 256, 0, stream, y, z, ld_z, w, eps, width, parts, (float*)out);
    else if (out_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(gated_group_norm_kernel<bf16>, grid, 256, 0, stream, y, z, ld_z, w, eps, width, parts, (bf16*)out);
    else
        return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}
