// Paged attention over pages that hold keys only, where a value is the leading part of its key row (bf16 cache).
//
// Two mixers cache that way: attention whose values are its keys (the whole row is the value), and latent
// attention, whose cached row is [latent | rotated key part] shared by all heads and whose value sum is taken over
// the latent, which the caller expands per head afterwards.  Both may have many query heads on one key head, row
// sizes up to 512 elements, and two further rules for the scores:
//   keep_first   under the window mask, the first `keep_first` positions of a sequence stay visible;
//   dist_bias    [far + 1, nq] floats: dist_bias[min(pos - key, far), head] is added to the scaled score.
//
//   keys_prefill_kernel   one CTA = one query head, one tile of up to 64 consecutive rows of one request (the tile
//                         list of the other prefill kernels), one chunk of up to 256 value columns.  It walks the key
//                         blocks (64 keys, at absolute multiples of 64) that hold kept positions and then those from
//                         the tile's lowest visible key on: cp.async into two stages, Q K^T and P V on the tensor
//                         cores (m16n8k16) with the online softmax in float32 registers.  The row size is a run-time
//                         multiple of 16 (the query fragments are re-read from shared memory), the value chunk a
//                         template parameter (its accumulators live in registers).
//   keys_decode_kernel    one CTA = one row that brings a single query, one group of up to 16 query heads of one key
//                         head (they are the 16 rows of the MMA, so a key is read once for all of them), one split of
//                         256 keys at an absolute multiple of 256, one value chunk; its four warps take 16 keys each
//                         of every block of 64.  It leaves an unnormalised partial (max, sum, weighted values);
//   keys_decode_warp_kernel   the same CTA where shared memory holds a split's 256 keys twice an SM: a warp owns one
//                         block of 64 keys, asks for it at once and takes it in one pass;
//   keys_merge_kernel     adds a row's partials in the order of the splits.
// Blocks and splits sit at absolute positions and are added in ascending order, so a row's result depends on its
// position and keys alone, not on how a prompt was cut or on the rest of the batch.
#include "common.cuh"
#include "mma_sync.cuh"

using namespace mma16;

constexpr int KA_BQ = 64;         // query rows a prefill CTA
constexpr int KA_BK = 64;         // keys a block
constexpr int KA_THREADS = 128;
constexpr int KA_SPLIT = 256;     // keys a decode CTA
constexpr float KA_LOG2E = 1.4426950408889634f;

struct KeysArgs {
    const bf16* q;            // [T, nq, D]
    const bf16* kv;           // [pages, 1, nkv, page_size, D]
    const int* block_table;   // [B, max_blocks]
    const int* tiles;         // prefill: [n_tiles, 4]: first row, rows, first position, request index
    const int* row_req;       // decode: [T]
    const int* positions;     // decode: [T]
    const int* rows;          // decode: [R] rows served, or null for rows 0 .. R-1
    const float* dist_bias;   // [dist_far + 1, nq] or null
    float* part_o;            // decode: [R, nq, max_splits, dv]
    float* part_ml;           // decode: [R, nq, max_splits, 2]   (max in log2 units, sum)
    bf16* out;                // [T, nq, dv]
    int nq, nkv, D, dv, ld, max_blocks, page_size, page_shift, mask_kind, mask_span, keep_first, dist_far, max_splits;
    float scale_log2;
};

// Rows first, first + step, ... (`count` of them, at most 32) of the keys from key0 on into k_s, by one warp.  Its
// lanes first look up the places of the rows side by side (one wait for the block table, not one a row), then hand
// them round by shuffle; rows of up to 16 pieces of 16 bytes go two at a time, so that every lane copies.  No
// address needs a division by a run-time size.
__device__ __forceinline__ void keys_load_rows(const KeysArgs& a, const int* table, int kvh, int key0, int key_hi,
                                               bf16* k_s, int first, int step, int count) {
    const int vec = a.D >> 3;
    const int lane = threadIdx.x & 31;
    long long my_src = -1;                            // the element offset of row first + step * lane, -1: no such key
    if (lane < count) {
        const int key = key0 + first + step * lane;
        if (key <= key_hi) {
            const int blk = a.page_shift >= 0 ? (key >> a.page_shift) : (key / a.page_size);
            const int page = table[blk];
            if (page >= 0) my_src = (((long long)page * a.nkv + kvh) * a.page_size + (key - blk * a.page_size)) * a.D;
        }
    }
    if (vec <= 16) {
        const int half = lane >> 4, c = lane & 15;
        for (int i = 0; i < count; i += 2) {           // count is even
            const long long src = __shfl_sync(0xffffffffu, my_src, i + half);
            bf16* dst = k_s + (first + step * (i + half)) * a.ld;
            if (c < vec) cp_async_16(dst + c * 8, src >= 0 ? a.kv + src + c * 8 : a.kv, src >= 0 ? 16 : 0);
        }
    } else {
        for (int i = 0; i < count; ++i) {
            const long long src = __shfl_sync(0xffffffffu, my_src, i);
            bf16* dst = k_s + (first + step * i) * a.ld;
            for (int c = lane; c < vec; c += 32) cp_async_16(dst + c * 8, src >= 0 ? a.kv + src + c * 8 : a.kv, src >= 0 ? 16 : 0);
        }
    }
}

// One block of 64 keys into shared memory by all warps of the CTA: a warp takes every n-th row.
__device__ __forceinline__ void keys_load_block(const KeysArgs& a, const int* table, int kvh, int key0, int key_hi,
                                                bf16* k_s) {
    const int n_warps = blockDim.x >> 5;
    keys_load_rows(a, table, kvh, key0, key_hi, k_s, threadIdx.x >> 5, n_warps, KA_BK / n_warps);
}

// The scaled, biased and masked scores of one thread's part of a 16 x (8 NT) score tile, the running max and sum,
// and the correction of what was accumulated before.  Rows lane/4 (h = 0) and lane/4 + 8 (h = 1).
template <int NT>
__device__ __forceinline__ void keys_softmax_step(float (&s)[NT][4], int key0, const int (&pos_r)[2], const int (&lo_r)[2],
                                                  const int (&head_r)[2], int key_max, const KeysArgs& a,
                                                  const float* bias_s, int bias_ld, float (&m_run)[2], float (&l_run)[2],
                                                  float (&corr)[2], int lane) {
    float m_c[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int key = key0 + nt * 8 + (lane % 4) * 2 + (e & 1);
            const int h = e >> 1;
            const bool valid = key <= pos_r[h] && key <= key_max && (key >= lo_r[h] || key < a.keep_first);
            float v = s[nt][e] * a.scale_log2;
            if (bias_s != nullptr && valid) v += bias_s[min(pos_r[h] - key, a.dist_far) * bias_ld + head_r[h]] * KA_LOG2E;
            s[nt][e] = valid ? v : -INFINITY;
            m_c[h] = fmaxf(m_c[h], s[nt][e]);
        }
    float l_c[2] = {0.0f, 0.0f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        m_c[h] = fmaxf(m_c[h], __shfl_xor_sync(0xffffffffu, m_c[h], 1));
        m_c[h] = fmaxf(m_c[h], __shfl_xor_sync(0xffffffffu, m_c[h], 2));
        const float m_new = fmaxf(m_run[h], m_c[h]);
        corr[h] = (m_run[h] == -INFINITY) ? 0.0f : exp2f(m_run[h] - m_new);
        m_run[h] = m_new;
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = (s[nt][e] == -INFINITY) ? 0.0f : exp2f(s[nt][e] - m_run[e >> 1]);
            s[nt][e] = p;
            l_c[e >> 1] += p;
        }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_c[h] += __shfl_xor_sync(0xffffffffu, l_c[h], 1);
        l_c[h] += __shfl_xor_sync(0xffffffffu, l_c[h], 2);
        l_run[h] = l_run[h] * corr[h] + l_c[h];
    }
}

// S (16 x 8 NT) = Q (16 x D, rows q_rows of q_s) K^T (keys k_row0 .. of k_s), D a run-time multiple of 16
template <int NT>
__device__ __forceinline__ void keys_scores(float (&s)[NT][4], const bf16* q_s, const bf16* k_s, int k_row0, int D, int ld,
                                            int lane) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
    const bf16* q_at = q_s + (lane % 16) * ld + (lane / 16) * 8;
    const int pairs = D / 32;
    for (int k2 = 0; k2 < pairs; ++k2) {
        uint32_t qa0[4], qa1[4];
        ldmatrix_x4(qa0, q_at + k2 * 32);
        ldmatrix_x4(qa1, q_at + k2 * 32 + 16);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint32_t b[4];
            ldmatrix_x4(b, k_s + (k_row0 + nt * 8 + (lane % 8)) * ld + k2 * 32 + (lane / 8) * 8);
            mma_bf16(s[nt], qa0, b[0], b[1]);
            mma_bf16(s[nt], qa1, b[2], b[3]);
        }
    }
    if (D % 32 != 0) {
        uint32_t qa[4];
        ldmatrix_x4(qa, q_at + (D - 16));
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            uint32_t b[2];
            ldmatrix_x2(b, k_s + (k_row0 + nt * 8 + (lane % 8)) * ld + (D - 16) + ((lane / 8) % 2) * 8);
            mma_bf16(s[nt], qa, b[0], b[1]);
        }
    }
}

template <int NV, int HPC>     // value columns a CTA: 16 NV; query heads a CTA (of one key head): four warps each
__global__ void __launch_bounds__(KA_THREADS * HPC) keys_prefill_kernel(KeysArgs a) {
    extern __shared__ __align__(16) uint8_t smem_bytes[];
    const int ld = a.ld;
    bf16* q_s = reinterpret_cast<bf16*>(smem_bytes);      // [HPC][64][ld]
    bf16* kv_s = q_s + HPC * KA_BQ * ld;                    // [2 stages][64][ld]
    float* bias_s = reinterpret_cast<float*>(kv_s + 2 * KA_BK * ld);     // [HPC][dist_far + 1]: the heads' columns

    const int warp = (threadIdx.x >> 5) % 4, lane = threadIdx.x & 31, hi = threadIdx.x / KA_THREADS;
    const int* tile = a.tiles + (size_t)(gridDim.y - 1 - blockIdx.y) * 4;      // the tiles with the most keys first
    const int row0 = tile[0], n_rows = tile[1], p0 = tile[2];
    const int* table = a.block_table + (size_t)tile[3] * a.max_blocks;
    const int head = blockIdx.x * HPC + hi;
    const int kvh = head / (a.nq / a.nkv);
    const int vcol0 = blockIdx.z * (16 * NV);
    q_s += hi * KA_BQ * ld;
    bias_s += hi * (a.dist_far + 1);
    const int tid = threadIdx.x % KA_THREADS;

    const int p_last = p0 + n_rows - 1;
    const int key_lo = visible_lo(p0, a.mask_kind, a.mask_span);
    const int kb_first = key_lo / KA_BK, kb_last = p_last / KA_BK;
    // key blocks that hold kept positions and lie wholly below the first block of the window
    const int keep = a.mask_kind == SHARPI_MASK_WINDOW ? a.keep_first : 0;
    const int n_keep = min((keep + KA_BK - 1) / KA_BK, kb_first);
    const int n_iter = n_keep + (kb_last - kb_first + 1);
    auto block_of = [&](int it) { return it < n_keep ? it : kb_first + (it - n_keep); };

    const int vec = a.D / 8;
    for (int r = warp; r < KA_BQ; r += 4) {
        const bool valid = r < n_rows;
        const bf16* src = valid ? a.q + ((size_t)(row0 + r) * a.nq + head) * a.D : a.q;
        for (int c = lane; c < vec; c += 32) cp_async_16(q_s + r * ld + c * 8, valid ? src + c * 8 : src, valid ? 16 : 0);
    }
    keys_load_block(a, table, kvh, block_of(0) * KA_BK, p_last, kv_s);
    cp_async_commit();
    if (a.dist_bias != nullptr)
        for (int i = tid; i <= a.dist_far; i += KA_THREADS) bias_s[i] = a.dist_bias[(size_t)i * a.nq + head];

    float o[2 * NV][4];
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    int pos_r[2], lo_r[2];
    const int head_r[2] = {0, 0};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        pos_r[h] = p0 + warp * 16 + lane / 4 + 8 * h;
        lo_r[h] = visible_lo(pos_r[h], a.mask_kind, a.mask_span);
    }
    const int warp_pos_hi = p0 + warp * 16 + 15;

    for (int it = 0; it < n_iter; ++it) {
        const int stage = it & 1;
        bf16* k_s = kv_s + (size_t)stage * KA_BK * ld;
        if (it + 1 < n_iter) {
            keys_load_block(a, table, kvh, block_of(it + 1) * KA_BK, p_last, kv_s + (size_t)(stage ^ 1) * KA_BK * ld);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key0 = block_of(it) * KA_BK;
        if (key0 <= warp_pos_hi && warp * 16 < n_rows) {
            float s[KA_BK / 8][4];
            keys_scores<KA_BK / 8>(s, q_s + warp * 16 * ld, k_s, 0, a.D, ld, lane);
            float corr[2];
            keys_softmax_step<KA_BK / 8>(s, key0, pos_r, lo_r, head_r, p_last, a, a.dist_bias ? bias_s : nullptr, 1, m_run,
                                         l_run, corr, lane);
#pragma unroll
            for (int i = 0; i < 2 * NV; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int j = 0; j < KA_BK / 16; ++j) {
                uint32_t pa[4];
                pa[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
                pa[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
                pa[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
                pa[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
                for (int d2 = 0; d2 < NV; ++d2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, k_s + (j * 16 + (lane % 8) + ((lane / 8) % 2) * 8) * ld + vcol0 + d2 * 16 + (lane / 16) * 8);
                    mma_bf16(o[2 * d2], pa, b[0], b[1]);
                    mma_bf16(o[2 * d2 + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = warp * 16 + lane / 4 + 8 * h;
        if (r < n_rows) {
            const float inv = 1.0f / l_run[h];
            bf16* dst = a.out + ((size_t)(row0 + r) * a.nq + head) * a.dv;
#pragma unroll
            for (int i = 0; i < 2 * NV; ++i) {
                const int col = vcol0 + i * 8 + (lane % 4) * 2;
                if (col < a.dv)
                    *reinterpret_cast<__nv_bfloat162*>(dst + col) = __floats2bfloat162_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
            }
        }
    }
}

// The end of a decode CTA: every warp leaves its partial in shared memory (the key blocks are no longer read), then
// the block adds the four in the order of the warps and writes the split's partial.
template <int NV>
__device__ __forceinline__ void keys_decode_finish(const KeysArgs& a, bf16* kv_s, const float (&o)[2 * NV][4],
                                                   const float (&m_run)[2], const float (&l_run)[2], int heads_here,
                                                   int head0, int vcol0, int ri, int split, int chunk) {
    constexpr int DVC = 16 * NV;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* o_w = reinterpret_cast<float*>(kv_s) + (size_t)warp * (16 * DVC + 32);     // [16][DVC] then [16][2]
    float* ml_w = o_w + 16 * DVC;
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o_w[(lane / 4 + 8 * (e >> 1)) * DVC + i * 8 + (lane % 4) * 2 + (e & 1)] = o[i][e];
    if (lane % 4 == 0) {
        ml_w[(lane / 4) * 2] = m_run[0];
        ml_w[(lane / 4) * 2 + 1] = l_run[0];
        ml_w[(lane / 4 + 8) * 2] = m_run[1];
        ml_w[(lane / 4 + 8) * 2 + 1] = l_run[1];
    }
    __syncthreads();
    const float* base = reinterpret_cast<const float*>(kv_s);
    constexpr int WS = 16 * DVC + 32;
    for (int idx = threadIdx.x; idx < heads_here * DVC; idx += KA_THREADS) {
        const int g = idx / DVC, dd = idx % DVC;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, base[w * WS + 16 * DVC + g * 2]);
        float acc = 0.0f, L = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = base[w * WS + 16 * DVC + g * 2];
            const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
            acc += f * base[w * WS + g * DVC + dd];
            L += f * base[w * WS + 16 * DVC + g * 2 + 1];
        }
        const size_t slot = ((size_t)ri * a.nq + head0 + g) * a.max_splits + split;
        if (vcol0 + dd < a.dv) a.part_o[slot * a.dv + vcol0 + dd] = acc;
        if (dd == 0 && chunk == 0) {
            a.part_ml[slot * 2] = M;
            a.part_ml[slot * 2 + 1] = L;
        }
    }
}

// The same CTA with a block of 64 keys a warp: every warp asks for its whole block at once, waits once and takes the
// 64 keys in one pass (one maximum, no correction of earlier sums, the query fragments read once), and nothing but
// the query tile and the end is shared between the warps.  Shared memory holds the split's 256 keys; sizes that
// leave room for fewer than two CTAs an SM take keys_decode_kernel.
template <int NV>
__global__ void __launch_bounds__(KA_THREADS) keys_decode_warp_kernel(KeysArgs a) {
    extern __shared__ __align__(16) uint8_t smem_bytes[];
    const int ld = a.ld;
    bf16* kv_s = reinterpret_cast<bf16*>(smem_bytes);     // [4 warps][64][ld]; the warps' partials afterwards
    bf16* q_s = kv_s + 4 * KA_BK * ld;                      // [16][ld]
    constexpr int DVC = 16 * NV;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    const int G = a.nq / a.nkv;
    const int groups = (G + 15) / 16;
    const int n_chunks = gridDim.y / (a.nkv * groups);
    const int chunk = blockIdx.y % n_chunks;
    const int kvh = (blockIdx.y / n_chunks) / groups, hg = (blockIdx.y / n_chunks) % groups;
    const int head0 = kvh * G + hg * 16;
    const int heads_here = min(16, G - hg * 16);
    const int vcol0 = chunk * DVC;
    const int ri = blockIdx.z, split = blockIdx.x;
    const int r = a.rows ? a.rows[ri] : ri;
    const int pos = a.positions[r];
    const int lo = visible_lo(pos, a.mask_kind, a.mask_span);
    const int keep = a.mask_kind == SHARPI_MASK_WINDOW ? a.keep_first : 0;
    const int k0 = split * KA_SPLIT;
    if (k0 > pos) return;                                     // the merge reads the splits up to pos / 256 only
    const int k1 = min(pos, k0 + KA_SPLIT - 1);
    if (k1 < lo && k0 >= keep) {                              // a split wholly behind the window: an empty partial
        if (chunk == 0 && threadIdx.x < heads_here) {
            const size_t slot = ((size_t)ri * a.nq + head0 + threadIdx.x) * a.max_splits + split;
            a.part_ml[slot * 2] = -INFINITY;
            a.part_ml[slot * 2 + 1] = 0.0f;
        }
        return;
    }
    const int b0 = k0 + warp * KA_BK;                         // this warp's block
    const bool mine = b0 <= k1 && (min(k1, b0 + KA_BK - 1) >= lo || b0 < keep);
    bf16* k_s = kv_s + (size_t)warp * KA_BK * ld;
    if (mine) {
        const int* table = a.block_table + (size_t)a.row_req[r] * a.max_blocks;
        keys_load_rows(a, table, kvh, b0, k1, k_s, 0, 1, 32);
        keys_load_rows(a, table, kvh, b0, k1, k_s, 32, 1, 32);
    }
    cp_async_commit();
    const int vec = a.D / 8;
    for (int g = warp; g < 16; g += 4)
        for (int c = lane; c < vec; c += 32) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (g < heads_here) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)r * a.nq + head0 + g) * a.D + c * 8);
            *reinterpret_cast<uint4*>(q_s + g * ld + c * 8) = v;
        }

    float o[2 * NV][4];
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const int pos_r[2] = {pos, pos}, lo_r[2] = {lo, lo};
    const int head_r[2] = {min(head0 + lane / 4, a.nq - 1), min(head0 + lane / 4 + 8, a.nq - 1)};
    cp_async_wait<0>();
    __syncthreads();                    // the query tile and every warp's own keys are in shared memory
    if (mine) {
        float s[KA_BK / 8][4];
        keys_scores<KA_BK / 8>(s, q_s, k_s, 0, a.D, ld, lane);
        float corr[2];                  // of nothing: this is the warp's only pass
        keys_softmax_step<KA_BK / 8>(s, b0, pos_r, lo_r, head_r, k1, a, a.dist_bias, a.nq, m_run, l_run, corr, lane);
#pragma unroll
        for (int j = 0; j < KA_BK / 16; ++j) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
            pa[1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
            pa[2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
            pa[3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < NV; ++d2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, k_s + (j * 16 + (lane % 8) + ((lane / 8) % 2) * 8) * ld + vcol0 + d2 * 16 + (lane / 16) * 8);
                mma_bf16(o[2 * d2], pa, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], pa, b[2], b[3]);
            }
        }
    }
    __syncthreads();                    // the key blocks are no longer read
    keys_decode_finish<NV>(a, kv_s, o, m_run, l_run, heads_here, head0, vcol0, ri, split, chunk);
}

template <int NV>
__global__ void __launch_bounds__(KA_THREADS) keys_decode_kernel(KeysArgs a) {
    extern __shared__ __align__(16) uint8_t smem_bytes[];
    const int ld = a.ld;
    bf16* kv_s = reinterpret_cast<bf16*>(smem_bytes);     // [2 stages][64][ld]; the warps' partials afterwards
    bf16* q_s = kv_s + 2 * KA_BK * ld;                      // [16][ld]
    constexpr int DVC = 16 * NV;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    const int G = a.nq / a.nkv;
    const int groups = (G + 15) / 16;
    const int n_chunks = gridDim.y / (a.nkv * groups);
    const int chunk = blockIdx.y % n_chunks;
    const int kvh = (blockIdx.y / n_chunks) / groups, hg = (blockIdx.y / n_chunks) % groups;
    const int head0 = kvh * G + hg * 16;
    const int heads_here = min(16, G - hg * 16);
    const int vcol0 = chunk * DVC;
    const int ri = blockIdx.z, split = blockIdx.x;
    const int r = a.rows ? a.rows[ri] : ri;
    const int pos = a.positions[r];
    const int lo = visible_lo(pos, a.mask_kind, a.mask_span);
    const int keep = a.mask_kind == SHARPI_MASK_WINDOW ? a.keep_first : 0;
    const int k0 = split * KA_SPLIT;
    if (k0 > pos) return;                                     // the merge reads the splits up to pos / 256 only
    const int k1 = min(pos, k0 + KA_SPLIT - 1);
    // blocks of 64 keys of this split that hold a visible key
    int live[KA_SPLIT / KA_BK], n_live = 0;
#pragma unroll
    for (int b = 0; b < KA_SPLIT / KA_BK; ++b) {
        const int b0 = k0 + b * KA_BK;
        if (b0 <= k1 && (min(k1, b0 + KA_BK - 1) >= lo || b0 < keep)) live[n_live++] = b0;
    }
    if (n_live == 0) {
        if (chunk == 0 && threadIdx.x < heads_here) {
            const size_t slot = ((size_t)ri * a.nq + head0 + threadIdx.x) * a.max_splits + split;
            a.part_ml[slot * 2] = -INFINITY;
            a.part_ml[slot * 2 + 1] = 0.0f;
        }
        return;
    }
    const int* table = a.block_table + (size_t)a.row_req[r] * a.max_blocks;
    keys_load_block(a, table, kvh, live[0], k1, kv_s);
    cp_async_commit();
    const int vec = a.D / 8;
    for (int idx = threadIdx.x; idx < 16 * vec; idx += KA_THREADS) {
        const int g = idx / vec, c = idx % vec;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < heads_here) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)r * a.nq + head0 + g) * a.D + c * 8);
        *reinterpret_cast<uint4*>(q_s + g * ld + c * 8) = v;
    }

    float o[2 * NV][4];
#pragma unroll
    for (int i = 0; i < 2 * NV; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const int pos_r[2] = {pos, pos}, lo_r[2] = {lo, lo};
    const int head_r[2] = {min(head0 + lane / 4, a.nq - 1), min(head0 + lane / 4 + 8, a.nq - 1)};

    for (int it = 0; it < n_live; ++it) {
        const int stage = it & 1;
        bf16* k_s = kv_s + (size_t)stage * KA_BK * ld;
        if (it + 1 < n_live) {
            keys_load_block(a, table, kvh, live[it + 1], k1, kv_s + (size_t)(stage ^ 1) * KA_BK * ld);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int key0 = live[it] + warp * 16;
        if (key0 <= k1 && (min(k1, key0 + 15) >= lo || key0 < keep)) {
            float s[2][4];
            keys_scores<2>(s, q_s, k_s, warp * 16, a.D, ld, lane);
            float corr[2];
            keys_softmax_step<2>(s, key0, pos_r, lo_r, head_r, k1, a, a.dist_bias, a.nq, m_run, l_run, corr, lane);
#pragma unroll
            for (int i = 0; i < 2 * NV; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
            uint32_t pa[4];
            pa[0] = pack_bf16(s[0][0], s[0][1]);
            pa[1] = pack_bf16(s[0][2], s[0][3]);
            pa[2] = pack_bf16(s[1][0], s[1][1]);
            pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
            for (int d2 = 0; d2 < NV; ++d2) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, k_s + (warp * 16 + (lane % 8) + ((lane / 8) % 2) * 8) * ld + vcol0 + d2 * 16 + (lane / 16) * 8);
                mma_bf16(o[2 * d2], pa, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();
    }
    keys_decode_finish<NV>(a, kv_s, o, m_run, l_run, heads_here, head0, vcol0, ri, split, chunk);
}

// One block per (row, query head): the row's partials of splits 0 .. pos / 256, weighted by exp2(max_s - max), added
// in the order of the splits and normalised.
__global__ void __launch_bounds__(KA_THREADS) keys_merge_kernel(KeysArgs a) {
    pdl_wait();
    const int ri = blockIdx.x, head = blockIdx.y;
    const int r = a.rows ? a.rows[ri] : ri;
    const int n_s = a.positions[r] / KA_SPLIT + 1;
    const size_t slot0 = ((size_t)ri * a.nq + head) * a.max_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_s; ++s) M = fmaxf(M, a.part_ml[(slot0 + s) * 2]);
    float L = 0.0f;
    for (int s = 0; s < n_s; ++s) {
        const float m = a.part_ml[(slot0 + s) * 2];
        if (m != -INFINITY) L += exp2f(m - M) * a.part_ml[(slot0 + s) * 2 + 1];
    }
    const float inv = 1.0f / L;
    for (int col = threadIdx.x; col < a.dv; col += KA_THREADS) {
        float acc = 0.0f;
        for (int s = 0; s < n_s; ++s) {
            const float m = a.part_ml[(slot0 + s) * 2];
            if (m != -INFINITY) acc += exp2f(m - M) * a.part_o[(slot0 + s) * a.dv + col];
        }
        a.out[((size_t)r * a.nq + head) * a.dv + col] = __float2bfloat16_rn(acc * inv);
    }
}

static bool keys_fill(KeysArgs& a, const void* q, const void* kv, const int* block_table, void* out, int nq, int nkv, int D,
                      int dv, int max_blocks, int page_size, int mask_kind, int mask_span, int keep_first,
                      const float* dist_bias, int dist_far, float scale, int* nv, int* n_chunks) {
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || page_size <= 0 || max_blocks <= 0 || nq > 65535) return false;
    if (D <= 0 || D % 16 != 0 || D > 512 || dv <= 0 || dv % 16 != 0 || dv > D) return false;
    if (mask_kind != SHARPI_MASK_FULL && mask_span <= 0) return false;
    if (keep_first < 0 || (dist_bias && dist_far < 0)) return false;
    a.q = (const bf16*)q; a.kv = (const bf16*)kv; a.block_table = block_table; a.out = (bf16*)out;
    a.tiles = nullptr; a.row_req = nullptr; a.positions = nullptr; a.rows = nullptr; a.part_o = nullptr; a.part_ml = nullptr;
    a.dist_bias = dist_bias; a.nq = nq; a.nkv = nkv; a.D = D; a.dv = dv; a.max_blocks = max_blocks; a.page_size = page_size;
    a.mask_kind = mask_kind; a.mask_span = mask_span; a.keep_first = keep_first; a.dist_far = dist_bias ? dist_far : 0;
    a.max_splits = 0; a.scale_log2 = scale * KA_LOG2E;
    a.page_shift = -1;
    for (int sft = 0; sft < 31; ++sft)
        if ((1 << sft) == page_size) a.page_shift = sft;
    *nv = dv <= 16 ? 1 : dv <= 32 ? 2 : dv <= 64 ? 4 : dv <= 128 ? 8 : 16;
    *n_chunks = (dv + 16 * *nv - 1) / (16 * *nv);
    const int cols = *n_chunks * 16 * *nv;
    a.ld = (D > cols ? D : cols) + 8;
    return true;
}

template <int NV, int HPC>
static int keys_launch_prefill_h(const KeysArgs& a, int n_tiles, int n_chunks, size_t smem, cudaStream_t stream) {
    static size_t configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(keys_prefill_kernel<NV, HPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return SHARPI_LAUNCH_FAILED;
        configured = smem;
    }
    keys_prefill_kernel<NV, HPC><<<dim3(a.nq / HPC, n_tiles, n_chunks), KA_THREADS * HPC, smem, stream>>>(a);
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// Two heads of one key head share a CTA (and its key blocks) where there are two and shared memory holds both query tiles.
template <int NV>
static int keys_launch_prefill(const KeysArgs& a, int n_tiles, int n_chunks, cudaStream_t stream) {
    const size_t bias = (size_t)(a.dist_far + 1) * 4;
    const size_t one = (size_t)3 * KA_BK * a.ld * 2 + bias, two = (size_t)4 * KA_BK * a.ld * 2 + 2 * bias;
    if (one > 227 * 1024) return SHARPI_BAD_ARGUMENT;
    if ((a.nq / a.nkv) % 2 == 0 && two <= 227 * 1024) return keys_launch_prefill_h<NV, 2>(a, n_tiles, n_chunks, two, stream);
    return keys_launch_prefill_h<NV, 1>(a, n_tiles, n_chunks, one, stream);
}

template <int NV>
static int keys_launch_decode(const KeysArgs& a, int R, int splits, int n_chunks, cudaStream_t stream) {
    const size_t smem = (size_t)(2 * KA_BK + 16) * a.ld * 2;
    static size_t configured = 0;
    if (smem > configured) {
        if (cudaFuncSetAttribute(keys_decode_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return SHARPI_LAUNCH_FAILED;
        configured = smem;
    }
    const int G = a.nq / a.nkv;
    const dim3 grid(splits, a.nkv * ((G + 15) / 16) * n_chunks, R);
    const size_t smem_warp = (size_t)(4 * KA_BK + 16) * a.ld * 2;
    if (smem_warp <= 113 * 1024) {
        static size_t configured_warp = 0;
        if (smem_warp > configured_warp) {
            if (cudaFuncSetAttribute(keys_decode_warp_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_warp) != cudaSuccess)
                return SHARPI_LAUNCH_FAILED;
            configured_warp = smem_warp;
        }
        auto kern = keys_decode_warp_kernel<NV>;
        SHARPI_LAUNCH_PDL(kern, grid, KA_THREADS, smem_warp, stream, a);
    } else {
        auto kern = keys_decode_kernel<NV>;
        SHARPI_LAUNCH_PDL(kern, grid, KA_THREADS, smem, stream, a);
    }
    SHARPI_LAUNCH_PDL(keys_merge_kernel, dim3(R, a.nq), KA_THREADS, 0, stream, a);
    return SHARPI_OK;
}

#define KEYS_DISPATCH(fn, ...)                         \
    switch (nv) {                                      \
        case 1: return fn<1>(__VA_ARGS__);             \
        case 2: return fn<2>(__VA_ARGS__);             \
        case 4: return fn<4>(__VA_ARGS__);             \
        case 8: return fn<8>(__VA_ARGS__);             \
        default: return fn<16>(__VA_ARGS__);           \
    }

// q [T, nq, D], out [T, nq, dv] bf16; the value of a key is the first dv elements of its row (dv a multiple of 16).
SHARPI_API int sharpi_attention_keys_prefill(const void* q, const void* kv, const int* block_table, const int* tiles,
                                             void* out, int n_tiles, int nq, int nkv, int D, int dv, int max_blocks,
                                             int page_size, int mask_kind, int mask_span, int keep_first,
                                             const float* dist_bias, int dist_far, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return SHARPI_OK;
    if (n_tiles > 65535) return SHARPI_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv) | reinterpret_cast<uintptr_t>(out)) & 15)
        return SHARPI_UNALIGNED;
    KeysArgs a;
    int nv, n_chunks;
    if (!keys_fill(a, q, kv, block_table, out, nq, nkv, D, dv, max_blocks, page_size, mask_kind, mask_span, keep_first,
                   dist_bias, dist_far, scale, &nv, &n_chunks))
        return SHARPI_BAD_ARGUMENT;
    a.tiles = tiles;
    KEYS_DISPATCH(keys_launch_prefill, a, n_tiles, n_chunks, stream)
}

// `splits`: at least (largest position of a served row) / 256 + 1; part_o / part_ml are scratch of
// [R, nq, splits, dv] and [R, nq, splits, 2] floats.
SHARPI_API int sharpi_attention_keys_decode(const void* q, const void* kv, const int* block_table, const int* row_req,
                                            const int* positions, const int* rows, float* part_o, float* part_ml,
                                            void* out, int R, int nq, int nkv, int D, int dv, int max_blocks,
                                            int page_size, int mask_kind, int mask_span, int keep_first,
                                            const float* dist_bias, int dist_far, int splits, float scale,
                                            cudaStream_t stream) {
    if (R <= 0) return SHARPI_OK;
    if (R > 65535 || splits <= 0) return SHARPI_BAD_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv)) & 15) return SHARPI_UNALIGNED;
    KeysArgs a;
    int nv, n_chunks;
    if (!keys_fill(a, q, kv, block_table, out, nq, nkv, D, dv, max_blocks, page_size, mask_kind, mask_span, keep_first,
                   dist_bias, dist_far, scale, &nv, &n_chunks))
        return SHARPI_BAD_ARGUMENT;
    a.row_req = row_req; a.positions = positions; a.rows = rows; a.part_o = part_o; a.part_ml = part_ml;
    a.max_splits = splits;
    KEYS_DISPATCH(keys_launch_decode, a, R, splits, n_chunks, stream)
}
