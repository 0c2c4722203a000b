// Latent attention around the paged attention kernels: keys and values are two readings of one cached latent.
//
// Per token the cache holds one row of D elements for all heads: [c (rank) | k_rot (rot) | zeros], c the
// RMS-normed latent and k_rot the rotated key part that every head shares.  A head's score is
// q_plain . (W_uk c) + q_rot . k_rot = (W_uk^T q_plain) . c + q_rot . k_rot, so a query row of a head is
// [W_uk^T q_plain | q_rot | zeros] and the attention kernels see one key/value head of size D whose value is the
// key row itself; of a head's output the first `rank` elements are sum_j p_j c_j, which W_uv then expands.
//
//   sharpi_latent_down_post  one block a token over the fused down projection [q latent | c | k_rot]:
//                            RMS norm with a weight of the q latent (-> activation dtype) and of c, rotation of
//                            k_rot by the token's position (pairs (2i, 2i + 1) of its first `rot_dims` elements),
//                            and the store of [c | k_rot | 0] into the token's place in the pages (and of
//                            [c | 0] into the value plane when a page has one).
//   sharpi_head_major        columns [col0, col0 + n) of every head of src [T, heads, stride] (float32 or the
//                            activation dtype) as dst [heads, T, n] in the activation dtype: the operand of a
//                            per-head (grouped) product.
//   sharpi_head_minor        the way back: src float32 [heads, T, n] into columns [col0, col0 + n) of
//                            dst [T, heads, stride] in the activation dtype.
//   sharpi_latent_q_join     the query rows: dst[t, h] = [qa[h, t, :rank] | rotate(q[t, h, dim:dim + rot]) | 0].
//
// `ld` / `ldq`: the distance between two rows of the source when it is a column range of a wider product; `rot_amp`:
// a factor on the rotation's cosines and sines (frequency scalings that also stretch the amplitude); `gate` of
// head_minor: [T, gate_ld] float32 logits, head h of row t is multiplied by sigmoid(gate[t, h]).
//
// Norm sums, angles, sines and cosines are float32; a row's numbers depend on the row alone.
#include "common.cuh"

constexpr int LAT_THREADS = 128;

template <typename TO>
__global__ void __launch_bounds__(LAT_THREADS)
latent_down_post_kernel(const float* down, int ld, int q_rank, int rank, int rot, int rot_dims,
                        const float* __restrict__ wq, const float* __restrict__ wc, float eps,
                        const int* positions, const int* row_req, const int* block_table, int max_blocks,
                        int page_size, const float* __restrict__ inv_freq, TO* cq_out, TO* kv_base, int kv_planes,
                        int D, int write_kv, float rot_amp) {
    __shared__ float scratch[32];
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = down + (size_t)t * ld;
    float ssq = 0.0f, ssc = 0.0f;
    for (int i = threadIdx.x; i < q_rank; i += LAT_THREADS) ssq += row[i] * row[i];
    for (int i = threadIdx.x; i < rank; i += LAT_THREADS) ssc += row[q_rank + i] * row[q_rank + i];
    ssq = block_sum(ssq, scratch);
    ssc = block_sum(ssc, scratch);
    if (q_rank > 0) {
        const float sq = 1.0f / sqrtf(ssq / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += LAT_THREADS)
            cq_out[(size_t)t * q_rank + i] = from_float<TO>(row[i] * sq * wq[i]);
    }
    if (!write_kv) return;
    const int pos = positions[t];
    const int page = block_table[(size_t)row_req[t] * max_blocks + pos / page_size];
    if (page < 0) return;   // the host checks before the launch that every written position has a page
    const size_t plane = (size_t)page_size * D;
    TO* krow = kv_base + (size_t)page * kv_planes * plane + (size_t)(pos % page_size) * D;
    TO* vrow = kv_planes == 2 ? krow + plane : nullptr;
    const float sc = 1.0f / sqrtf(ssc / (float)rank + eps);
    const float* kr = row + q_rank + rank;
    for (int i = threadIdx.x; i < D; i += LAT_THREADS) {
        float k = 0.0f, v = 0.0f;
        if (i < rank) {
            k = v = row[q_rank + i] * sc * wc[i];
        } else if (i < rank + rot) {
            const int j = i - rank;
            k = kr[j];
            if (j < rot_dims && inv_freq) {
                float sn, cs;
                sincosf((float)pos * inv_freq[j >> 1], &sn, &cs);
                sn *= rot_amp;
                cs *= rot_amp;
                k = (j & 1) ? kr[j] * cs + kr[j - 1] * sn : kr[j] * cs - kr[j + 1] * sn;
            }
        }
        krow[i] = from_float<TO>(k);
        if (vrow) vrow[i] = from_float<TO>(v);
    }
}

SHARPI_API int sharpi_latent_down_post(const float* down, int ld, int q_rank, int rank, int rot, int rot_dims,
                                       const float* wq, const float* wc, float eps, const int* positions,
                                       const int* row_req, const int* block_table, int max_blocks, int page_size,
                                       const float* inv_freq, void* cq_out, void* kv_base, int kv_planes, int D,
                                       int write_kv, int out_dtype, int T, float rot_amp, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (q_rank < 0 || rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) ||
        q_rank + rank + rot > ld || rank + rot > D || (kv_planes != 1 && kv_planes != 2) || page_size <= 0 ||
        max_blocks <= 0 || (q_rank > 0 && !wq) || !wc)
        return SHARPI_BAD_ARGUMENT;
    if (out_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(latent_down_post_kernel<float>, T, LAT_THREADS, 0, stream, down, ld, q_rank, rank, rot,
                          rot_dims, wq, wc, eps, positions, row_req, block_table, max_blocks, page_size, inv_freq,
                          (float*)cq_out, (float*)kv_base, kv_planes, D, write_kv, rot_amp);
    else if (out_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(latent_down_post_kernel<bf16>, T, LAT_THREADS, 0, stream, down, ld, q_rank, rank, rot,
                          rot_dims, wq, wc, eps, positions, row_req, block_table, max_blocks, page_size, inv_freq,
                          (bf16*)cq_out, (bf16*)kv_base, kv_planes, D, write_kv, rot_amp);
    else
        return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}

template <typename TS, typename TO>
__global__ void __launch_bounds__(256)
head_major_kernel(const TS* src, int T, int heads, int stride, int col0, int n, TO* dst, int ld) {
    pdl_wait();
    const long long total = (long long)T * heads * n;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = (int)(i % n);
    const long long th = i / n;
    const int t = (int)(th % T), h = (int)(th / T);
    dst[i] = from_float<TO>(to_float(src[(size_t)t * ld + (size_t)h * stride + col0 + c]));
}

SHARPI_API int sharpi_head_major(const void* src, int src_dtype, int T, int heads, int stride, int col0, int n,
                                 void* dst, int dst_dtype, int ld, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return SHARPI_OK;
    if (ld <= 0) ld = heads * stride;          // rows lie end to end
    if (heads <= 0 || col0 < 0 || col0 + n > stride || ld < heads * stride) return SHARPI_BAD_ARGUMENT;
    const long long total = (long long)T * heads * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (src_dtype == SHARPI_F32 && dst_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL((head_major_kernel<float, float>), blocks, 256, 0, stream, (const float*)src, T, heads, stride, col0, n, (float*)dst, ld);
    else if (src_dtype == SHARPI_F32 && dst_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL((head_major_kernel<float, bf16>), blocks, 256, 0, stream, (const float*)src, T, heads, stride, col0, n, (bf16*)dst, ld);
    else if (src_dtype == SHARPI_BF16 && dst_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL((head_major_kernel<bf16, bf16>), blocks, 256, 0, stream, (const bf16*)src, T, heads, stride, col0, n, (bf16*)dst, ld);
    else
        return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}

template <typename TO>
__global__ void __launch_bounds__(256)
head_minor_kernel(const float* src, int T, int heads, int stride, int col0, int n, TO* dst, const float* gate,
                  int gate_ld) {
    pdl_wait();
    const long long total = (long long)T * heads * n;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = (int)(i % n);
    const long long th = i / n;
    const int h = (int)(th % heads), t = (int)(th / heads);
    float v = src[((size_t)h * T + t) * n + c];
    if (gate) v = v / (1.0f + expf(-gate[(size_t)t * gate_ld + h]));      // the head's output times sigmoid(gate logit)
    dst[((size_t)t * heads + h) * stride + col0 + c] = from_float<TO>(v);
}

SHARPI_API int sharpi_head_minor(const float* src, int T, int heads, int stride, int col0, int n, void* dst,
                                 int dst_dtype, const float* gate, int gate_ld, cudaStream_t stream) {
    if (T <= 0 || n <= 0) return SHARPI_OK;
    if (heads <= 0 || col0 < 0 || col0 + n > stride) return SHARPI_BAD_ARGUMENT;
    const long long total = (long long)T * heads * n;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dst_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(head_minor_kernel<float>, blocks, 256, 0, stream, src, T, heads, stride, col0, n, (float*)dst, gate, gate_ld);
    else if (dst_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(head_minor_kernel<bf16>, blocks, 256, 0, stream, src, T, heads, stride, col0, n, (bf16*)dst, gate, gate_ld);
    else
        return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}

template <typename TO>
__global__ void __launch_bounds__(256)
latent_q_join_kernel(const float* qa, const float* q, const int* positions, const float* __restrict__ inv_freq, int T,
                     int heads, int dim, int rank, int rot, int rot_dims, int D, TO* dst, int ldq, float rot_amp) {
    pdl_wait();
    const long long total = (long long)T * heads * D;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = (int)(i % D);
    const long long th = i / D;
    const int h = (int)(th % heads), t = (int)(th / heads);
    float v = 0.0f;
    if (c < rank) {
        v = qa[((size_t)h * T + t) * rank + c];
    } else if (c < rank + rot) {
        const int j = c - rank;
        const float* qr = q + (size_t)t * ldq + (size_t)h * (dim + rot) + dim;
        v = qr[j];
        if (j < rot_dims && inv_freq) {
            float sn, cs;
            sincosf((float)positions[t] * inv_freq[j >> 1], &sn, &cs);
            sn *= rot_amp;
            cs *= rot_amp;
            v = (j & 1) ? qr[j] * cs + qr[j - 1] * sn : qr[j] * cs - qr[j + 1] * sn;
        }
    }
    dst[i] = from_float<TO>(v);
}

SHARPI_API int sharpi_latent_q_join(const float* qa, const float* q, const int* positions, const float* inv_freq,
                                    int T, int heads, int dim, int rank, int rot, int rot_dims, int D, void* dst,
                                    int dst_dtype, int ldq, float rot_amp, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (ldq <= 0) ldq = heads * (dim + rot);   // rows lie end to end
    if (heads <= 0 || dim <= 0 || rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) ||
        rank + rot > D)
        return SHARPI_BAD_ARGUMENT;
    const long long total = (long long)T * heads * D;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dst_dtype == SHARPI_F32)
        SHARPI_LAUNCH_PDL(latent_q_join_kernel<float>, blocks, 256, 0, stream, qa, q, positions, inv_freq, T, heads,
                          dim, rank, rot, rot_dims, D, (float*)dst, ldq, rot_amp);
    else if (dst_dtype == SHARPI_BF16)
        SHARPI_LAUNCH_PDL(latent_q_join_kernel<bf16>, blocks, 256, 0, stream, qa, q, positions, inv_freq, T, heads,
                          dim, rank, rot, rot_dims, D, (bf16*)dst, ldq, rot_amp);
    else
        return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}
