// The state-space-duality recurrence (Mamba-2) from per-request state, walked row by row, and the gated norm in
// groups behind it.
//
//   sharpi_ssd_scan     per head h (its group g = h / (heads / groups)), for the rows of a request in order:
//                         dt = softplus(dt_raw[h] + dt_bias[h]);  a = exp(-exp(A_log[h]) * dt)
//                         S[n][v] <- a S[n][v] + dt B_g[n] x_h[v]        (S is N x P per head, float32)
//                         y_h[v]  = sum_n S[n][v] C_g[n] + D[h] x_h[v]
//                       x, B and C are columns of one float32 matrix (the convolution's output), dt_raw columns of
//                       another (the fused input projection).  A block serves one (request, head, 32 value columns);
//                       eight lanes share a column, each keeping N / 8 of its states in registers (lane l holds the
//                       states 32 j + 4 l .. + 3, so that it reads B and C four at a time without bank conflicts).
//                       The rows come in chunks of SSD_CH through three shared-memory buffers filled by cp.async, two
//                       chunks ahead of the walk, so that the walk never waits for memory after its first chunk.  The
//                       sum over the states is a fixed order inside a lane and a fixed tree across the eight lanes,
//                       and the walk over a request's rows is sequential, so a row's result does not depend on how a
//                       prompt was cut or batched.  The state is read at the start of a portion and stored behind
//                       its last row.
//   sharpi_gated_group_norm   u = y * silu(z);  out = u / sqrt(mean_part(u^2) + eps) * w, the width in `parts` equal
//                       consecutive parts, each with its own mean (float32; output in the activation dtype).
#include "common.cuh"
#include "mma_sync.cuh"

constexpr int SSD_THREADS = 256;
constexpr int SSD_LANES = 8;                         // lanes that share one value column
constexpr int SSD_COLS = SSD_THREADS / SSD_LANES;    // value columns a block
constexpr int SSD_CH = 16;                           // rows staged together
constexpr int SSD_STAGES = 3;
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
    int walk;                // some request brings more than one row: launched the plain way, onto an empty GPU
};

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(mma16::smem_addr(smem_dst)), "l"(gmem_src) : "memory");
}

template <int NPL>           // states a lane; the rows of B and C in shared memory hold NP = 8 NPL floats (zeros behind N)
__global__ void __launch_bounds__(SSD_THREADS) ssd_scan_kernel(SsdArgs a) {
    constexpr int NP = SSD_LANES * NPL;
    constexpr int STAGE = SSD_CH * (2 * NP + SSD_COLS + 2);      // floats: B, C, x, raw dt then dt, decay
    extern __shared__ __align__(16) float smem[];
    const int N = a.N, P = a.P;
    if (a.walk) pdl_wait_only(); else pdl_wait();
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
        const int n = 32 * (j / 4) + 4 * lane + (j % 4);
        S[j] = (live && n < N) ? st[(size_t)n * P + v] : 0.0f;
    }
    // what cp.async never writes is zero: states behind N, value columns behind P (where there are any: a block that
    // serves a single row would otherwise spend a third of its instructions here)
    if (N < NP || (blockIdx.x + 1) * SSD_COLS > P) {
        for (int i = threadIdx.x; i < SSD_STAGES * STAGE; i += SSD_THREADS) smem[i] = 0.0f;
        __syncthreads();
    }
    const bool vec = (N % 4 == 0) && (a.ld_x % 4 == 0) && ((a.col_b + g * N) % 4 == 0) && ((a.col_c + g * N) % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(a.xbc) & 15) == 0);
    const int n_chunks = (rows + SSD_CH - 1) / SSD_CH;
    auto issue = [&](int c) {
        if (c < n_chunks) {
            float* b_s = smem + (c % SSD_STAGES) * STAGE;
            float* c_s = b_s + SSD_CH * NP;
            float* x_s = c_s + SSD_CH * NP;
            float* d_s = x_s + SSD_CH * SSD_COLS;
            const int r0 = c * SSD_CH, nr = min(SSD_CH, rows - r0);
            if (vec) {
                const int per = N / 4;
                for (int i = threadIdx.x; i < nr * per; i += SSD_THREADS) {
                    const int r = i / per, q = i % per;
                    const float* row = a.xbc + (size_t)(first + r0 + r) * a.ld_x;
                    mma16::cp_async_16(b_s + r * NP + 4 * q, row + a.col_b + g * N + 4 * q, 16);
                    mma16::cp_async_16(c_s + r * NP + 4 * q, row + a.col_c + g * N + 4 * q, 16);
                }
            } else {
                for (int i = threadIdx.x; i < nr * N; i += SSD_THREADS) {
                    const int r = i / N, n = i % N;
                    const float* row = a.xbc + (size_t)(first + r0 + r) * a.ld_x;
                    cp_async_4(b_s + r * NP + n, row + a.col_b + g * N + n);
                    cp_async_4(c_s + r * NP + n, row + a.col_c + g * N + n);
                }
            }
            for (int i = threadIdx.x; i < nr * SSD_COLS; i += SSD_THREADS) {
                const int r = i / SSD_COLS, cc = i % SSD_COLS;
                const int vv = blockIdx.x * SSD_COLS + cc;
                if (vv < P) cp_async_4(x_s + i, a.xbc + (size_t)(first + r0 + r) * a.ld_x + a.col_x + h * P + vv);
            }
            if (threadIdx.x < nr) cp_async_4(d_s + threadIdx.x, a.dt + (size_t)(first + r0 + threadIdx.x) * a.ld_dt + a.col_dt + h);
        }
        mma16::cp_async_commit();        // a group every time, so that the count of groups in flight is fixed
    };
    const float decay_rate = -expf(a.a_log[h]);
    const float bias = a.dt_bias[h], dsk = a.dskip[h];
    issue(0);
    issue(1);
    for (int c = 0; c < n_chunks; ++c) {
        const int r0 = c * SSD_CH, nr = min(SSD_CH, rows - r0);
        mma16::cp_async_wait<1>();          // chunk c has landed (chunk c + 1 may be in flight)
        __syncthreads();                    // ... for every thread, and chunk c - 1 is no longer read
        issue(c + 2);                       // into the buffer of chunk c - 1
        float* b_s = smem + (c % SSD_STAGES) * STAGE;
        float* c_s = b_s + SSD_CH * NP;
        float* x_s = c_s + SSD_CH * NP;
        float* d_s = x_s + SSD_CH * SSD_COLS;
        if (threadIdx.x < nr) {
            const float d = softplus_f(d_s[threadIdx.x] + bias);
            d_s[threadIdx.x] = d;
            d_s[SSD_CH + threadIdx.x] = expf(decay_rate * d);
        }
        __syncthreads();
        for (int r = 0; r < nr; ++r) {
            const float d = d_s[r], decay = d_s[SSD_CH + r];
            const float xv = x_s[r * SSD_COLS + col];
            const float dx = d * xv;
            float acc = 0.0f;
#pragma unroll
            for (int j4 = 0; j4 < NPL / 4; ++j4) {
                const float4 bv = *reinterpret_cast<const float4*>(b_s + r * NP + 32 * j4 + 4 * lane);
                const float4 cv = *reinterpret_cast<const float4*>(c_s + r * NP + 32 * j4 + 4 * lane);
                S[4 * j4 + 0] = decay * S[4 * j4 + 0] + dx * bv.x; acc += S[4 * j4 + 0] * cv.x;
                S[4 * j4 + 1] = decay * S[4 * j4 + 1] + dx * bv.y; acc += S[4 * j4 + 1] * cv.y;
                S[4 * j4 + 2] = decay * S[4 * j4 + 2] + dx * bv.z; acc += S[4 * j4 + 2] * cv.z;
                S[4 * j4 + 3] = decay * S[4 * j4 + 3] + dx * bv.w; acc += S[4 * j4 + 3] * cv.w;
            }
#pragma unroll
            for (int o = SSD_LANES / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0 && live) a.y[(size_t)(first + r0 + r) * a.heads * P + h * P + v] = acc + dsk * xv;
        }
    }
    mma16::cp_async_wait<0>();
#pragma unroll
    for (int j = 0; j < NPL; ++j) {
        const int n = 32 * (j / 4) + 4 * lane + (j % 4);
        if (live && n < N) st[(size_t)n * P + v] = S[j];
    }
}

template <int NPL>
static int ssd_launch(const SsdArgs& a, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = (size_t)SSD_STAGES * SSD_CH * (2 * SSD_LANES * NPL + SSD_COLS + 2) * sizeof(float);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        if (cudaFuncSetAttribute(ssd_scan_kernel<NPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return SHARPI_LAUNCH_FAILED;
        configured = true;
    }
    auto kern = ssd_scan_kernel<NPL>;
    if (a.walk) {
        // a block walks its rows for hundreds of microseconds and there is less than a block an SM: started beside
        // the tail of the kernel before it, the blocks would share SMs that happened to be free and run at half speed
        kern<<<grid, SSD_THREADS, smem, stream>>>(a);
        SHARPI_CHECK_LAUNCH();
    } else {
        SHARPI_LAUNCH_PDL(kern, grid, SSD_THREADS, smem, stream, a);
    }
    return SHARPI_OK;
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
    a.groups = groups; a.N = N; a.P = P; a.walk = T > B;
    const dim3 grid((P + SSD_COLS - 1) / SSD_COLS, heads, B);
    const int per_lane = (N + SSD_LANES - 1) / SSD_LANES;
    if (per_lane <= 4) return ssd_launch<4>(a, grid, stream);
    if (per_lane <= 8) return ssd_launch<8>(a, grid, stream);
    if (per_lane <= 16) return ssd_launch<16>(a, grid, stream);
    return ssd_launch<32>(a, grid, stream);
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
