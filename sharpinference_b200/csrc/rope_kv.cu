// What happens to a fused Q|K|V projection before attention, in one pass over it:
// rotary position encoding of q and k, weightless L2 norm of q and k per head, the
// attention-temperature factor on q, the store of q for the attention kernel and the
// scatter of k and v into the pages of the cache.
//
// Reference order: RoPE, then the L2 norm, then the cache append
// (src/SharpInference.Engine/ForwardPass.cs:1635-1669); its CUDA path runs
// llm_rope_interleaved, llm_head_norm_pure and llm_kv_append one after the other
// (src/SharpInference.Cuda/CudaTextKernels.cs:653, :263, :850).  The temperature factor is
// not in the reference: q *= 1 + attn_scale * ln(1 + floor((pos + 1) / floor_scale)).
//
// Angles (pos * inv_freq), sin/cos, the norm's mean of squares and the temperature factor
// are fp32.  One warp owns one head of one token, so no result depends on the batch.  Head sizes
// that are multiples of four with interleaved pairs (or no rotation) take the kernel in which a lane
// owns whole 16-byte pieces, two pairs each; the others take the element-wise one.  Which of the two
// runs depends on the head size and the pairing alone.
#include "common.cuh"

enum RopePairing : int {
    ROPE_NONE = 0,
    ROPE_INTERLEAVED = 1,  // pairs (2j, 2j+1)
    ROPE_HALVES = 2,       // pairs (j, j + d/2)
};

struct QkvPostArgs {
    const float* qkv;        // [T, (nq + 2 nkv) * d]
    const int* positions;    // [T]
    const int* row_req;      // [T] index of the row's request in this step
    const int* block_table;  // [B, max_blocks] page ids of this layer's cache group
    const float* inv_freq;   // [d/2] or null
    void* q_out;             // [T, nq, d]
    void* kv_base;           // this layer's pages: [page][2][nkv][page_size][d]
    int T, nq, nkv, d;
    int max_blocks, page_size;
    int pairing;
    float l2_eps;            // < 0: no norm
    int l2_count;            // the mean of squares divides by this many elements (d, or fewer when the head
                             // is padded with zeros beyond its own size)
    float temp_attn_scale;   // temperature factor on q; floor_scale <= 0: none
    float temp_floor_scale;
    int write_kv;            // 0: this layer reads a cache that another layer writes
    int kv_planes;           // 2: q|k|v come in and a page holds [K|V]; 1: q|k come in and a page holds keys only
};

template <typename TO>
__global__ void qkv_post_kernel(QkvPostArgs a) {
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots = a.nq + a.kv_planes * a.nkv;
    const long long work = (long long)blockIdx.x * warps_per_block + warp;
    if (work >= (long long)a.T * slots) return;
    const int t = (int)(work / slots);
    const int slot = (int)(work % slots);
    const int d = a.d, half = d >> 1;
    const int pos = a.positions[t];
    const float* src = a.qkv + (size_t)t * slots * d + (size_t)slot * d;

    const bool is_q = slot < a.nq;
    const bool is_k = !is_q && slot < a.nq + a.nkv;
    const bool is_v = !is_q && !is_k;

    TO* dst;
    if (is_q) {
        dst = (TO*)a.q_out + ((size_t)t * a.nq + slot) * d;
    } else {
        if (!a.write_kv) return;
        const int head = is_k ? slot - a.nq : slot - a.nq - a.nkv;
        const int page = a.block_table[(size_t)a.row_req[t] * a.max_blocks + pos / a.page_size];
        if (page < 0) return;  // the host checks before the launch that every written position has a page
        const size_t plane = (size_t)a.nkv * a.page_size * d;
        dst = (TO*)a.kv_base + ((size_t)page * a.kv_planes + (is_k ? 0 : 1)) * plane +
              ((size_t)head * a.page_size + (pos % a.page_size)) * d;
    }

    if (is_v) {
        for (int i = lane; i < d; i += 32) dst[i] = from_float<TO>(src[i]);
        return;
    }

    // q or k: rotate, norm, scale.  A lane keeps its pairs in registers: up to 8 pairs per
    // lane covers head sizes up to 512.
    constexpr int MAX_PAIRS = 8;
    float x0[MAX_PAIRS], x1[MAX_PAIRS];
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < MAX_PAIRS; ++r) {
        const int j = lane + 32 * r;
        if (j < half) {
            const int i0 = (a.pairing == ROPE_HALVES) ? j : 2 * j;
            const int i1 = (a.pairing == ROPE_HALVES) ? j + half : 2 * j + 1;
            float v0 = src[i0], v1 = src[i1];
            if (a.pairing != ROPE_NONE && a.inv_freq) {
                const float angle = (float)pos * a.inv_freq[j];
                float sn, cs;
                sincosf(angle, &sn, &cs);
                const float r0 = v0 * cs - v1 * sn;
                const float r1 = v0 * sn + v1 * cs;
                v0 = r0;
                v1 = r1;
            }
            x0[r] = v0;
            x1[r] = v1;
            ss += v0 * v0 + v1 * v1;
        } else {
            x0[r] = 0.0f;
            x1[r] = 0.0f;
        }
    }
    float scale = 1.0f;
    if (a.l2_eps >= 0.0f) {
        ss = warp_sum(ss);
        scale = 1.0f / sqrtf(ss / (float)a.l2_count + a.l2_eps);
    }
    if (is_q && a.temp_floor_scale > 0.0f) {
        const float steps = floorf(((float)pos + 1.0f) / a.temp_floor_scale);
        scale *= 1.0f + a.temp_attn_scale * log1pf(steps);
    }
#pragma unroll
    for (int r = 0; r < MAX_PAIRS; ++r) {
        const int j = lane + 32 * r;
        if (j < half) {
            const int i0 = (a.pairing == ROPE_HALVES) ? j : 2 * j;
            const int i1 = (a.pairing == ROPE_HALVES) ? j + half : 2 * j + 1;
            dst[i0] = from_float<TO>(x0[r] * scale);
            dst[i1] = from_float<TO>(x1[r] * scale);
        }
    }
}

template <typename TO>
__device__ __forceinline__ void store4(TO* dst, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float4 v) {
    *reinterpret_cast<float4*>(dst) = v;
}
template <>
__device__ __forceinline__ void store4<bf16>(bf16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = w;
}

// d % 4 == 0, pairs (2j, 2j+1) or no rotation: lane l owns the four-element pieces l, l + 32, ... of a head.
// A warp serves QKV_SLOTS consecutive heads (q, k or v) of one token: their loads are issued together, and
// the sines and cosines of the lane's pairs, which depend on the token alone, are taken once.
constexpr int QKV_SLOTS = 4;

template <typename TO, int MAX_PIECES>      // MAX_PIECES * 128 >= head size
__global__ void __launch_bounds__(256) qkv_post_vec_kernel(QkvPostArgs a) {
    pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots = a.nq + a.kv_planes * a.nkv;
    const int groups = (slots + QKV_SLOTS - 1) / QKV_SLOTS;
    const long long work = (long long)blockIdx.x * warps_per_block + warp;
    if (work >= (long long)a.T * groups) return;
    const int t = (int)(work / groups);
    const int slot0 = (int)(work % groups) * QKV_SLOTS;
    const int d = a.d, n4 = d >> 2;
    float4 x[QKV_SLOTS][MAX_PIECES];
#pragma unroll
    for (int s = 0; s < QKV_SLOTS; ++s) {
        const float4* __restrict__ src =
            reinterpret_cast<const float4*>(a.qkv + (size_t)t * slots * d + (size_t)(slot0 + s) * d);
#pragma unroll
        for (int r = 0; r < MAX_PIECES; ++r) {
            const int i = lane + 32 * r;
            x[s][r] = (slot0 + s < slots && i < n4) ? src[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
    const int pos = a.positions[t];
    const bool rotate = a.pairing != ROPE_NONE && a.inv_freq;
    float cs0[MAX_PIECES], sn0[MAX_PIECES], cs1[MAX_PIECES], sn1[MAX_PIECES];
    if (rotate && slot0 < a.nq + a.nkv) {               // the group holds at least one q or k head
#pragma unroll
        for (int r = 0; r < MAX_PIECES; ++r) {
            const int i = lane + 32 * r;
            if (i < n4) {
                const float2 f = __ldg(reinterpret_cast<const float2*>(a.inv_freq) + i);   // pairs 2i, 2i + 1
                sincosf((float)pos * f.x, &sn0[r], &cs0[r]);
                sincosf((float)pos * f.y, &sn1[r], &cs1[r]);
            }
        }
    }
    // where this token's keys and values go
    int page = -1;
    if (a.write_kv && slot0 + QKV_SLOTS > a.nq)
        page = a.block_table[(size_t)a.row_req[t] * a.max_blocks + pos / a.page_size];
    const size_t plane = (size_t)a.nkv * a.page_size * d;
    float temp = 1.0f;
    if (a.temp_floor_scale > 0.0f && slot0 < a.nq) {
        const float steps = floorf(((float)pos + 1.0f) / a.temp_floor_scale);
        temp = 1.0f + a.temp_attn_scale * log1pf(steps);
    }
#pragma unroll
    for (int s = 0; s < QKV_SLOTS; ++s) {
        const int slot = slot0 + s;
        if (slot >= slots) break;
        const bool is_q = slot < a.nq;
        const bool is_k = !is_q && slot < a.nq + a.nkv;
        TO* dst;
        if (is_q) {
            dst = (TO*)a.q_out + ((size_t)t * a.nq + slot) * d;
        } else {
            if (page < 0) continue;      // no cache write for this layer (the host checks that written positions have pages)
            const int head = is_k ? slot - a.nq : slot - a.nq - a.nkv;
            dst = (TO*)a.kv_base + ((size_t)page * a.kv_planes + (is_k ? 0 : 1)) * plane +
                  ((size_t)head * a.page_size + (pos % a.page_size)) * d;
        }
        float scale = 1.0f;
        if (is_q || is_k) {
            float ss = 0.0f;
#pragma unroll
            for (int r = 0; r < MAX_PIECES; ++r) {
                const int i = lane + 32 * r;
                if (i < n4) {
                    if (rotate) {
                        const float4 v = x[s][r];
                        x[s][r] = make_float4(v.x * cs0[r] - v.y * sn0[r], v.x * sn0[r] + v.y * cs0[r],
                                              v.z * cs1[r] - v.w * sn1[r], v.z * sn1[r] + v.w * cs1[r]);
                    }
                    ss += x[s][r].x * x[s][r].x + x[s][r].y * x[s][r].y;
                    ss += x[s][r].z * x[s][r].z + x[s][r].w * x[s][r].w;
                }
            }
            if (a.l2_eps >= 0.0f) {
                ss = warp_sum(ss);
                scale = 1.0f / sqrtf(ss / (float)a.l2_count + a.l2_eps);
            }
            if (is_q) scale *= temp;
        }
#pragma unroll
        for (int r = 0; r < MAX_PIECES; ++r) {
            const int i = lane + 32 * r;
            if (i < n4)
                store4<TO>(dst + 4 * i, make_float4(x[s][r].x * scale, x[s][r].y * scale, x[s][r].z * scale, x[s][r].w * scale));
        }
    }
}

SHARPI_API int sharpi_qkv_post(const float* qkv, const int* positions, const int* row_req, const int* block_table,
                               const float* inv_freq, void* q_out, void* kv_base, int out_dtype, int T, int nq,
                               int nkv, int d, int max_blocks, int page_size, int pairing, float l2_eps,
                               float temp_attn_scale, float temp_floor_scale, int write_kv, int l2_count,
                               int kv_planes, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || (d & 1) || d > 512 || page_size <= 0 || max_blocks <= 0)
        return SHARPI_BAD_ARGUMENT;
    if (pairing != ROPE_NONE && pairing != ROPE_INTERLEAVED && pairing != ROPE_HALVES) return SHARPI_BAD_ARGUMENT;
    QkvPostArgs a;
    a.qkv = qkv; a.positions = positions; a.row_req = row_req; a.block_table = block_table;
    a.inv_freq = inv_freq; a.q_out = q_out; a.kv_base = kv_base;
    a.T = T; a.nq = nq; a.nkv = nkv; a.d = d; a.max_blocks = max_blocks; a.page_size = page_size;
    a.pairing = inv_freq ? pairing : ROPE_NONE; a.l2_eps = l2_eps;
    a.l2_count = (l2_count > 0 && l2_count <= d) ? l2_count : d;
    a.temp_attn_scale = temp_attn_scale; a.temp_floor_scale = temp_floor_scale; a.write_kv = write_kv;
    if (kv_planes != 1 && kv_planes != 2) return SHARPI_BAD_ARGUMENT;
    a.kv_planes = kv_planes;
    if (out_dtype != SHARPI_F32 && out_dtype != SHARPI_BF16) return SHARPI_BAD_ARGUMENT;
    const long long work = (long long)T * (nq + kv_planes * nkv);
    const long long vec_work = (long long)T * ((nq + kv_planes * nkv + QKV_SLOTS - 1) / QKV_SLOTS);
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                           reinterpret_cast<uintptr_t>(kv_base) | reinterpret_cast<uintptr_t>(inv_freq);
    if (d % 4 == 0 && a.pairing != ROPE_HALVES && (ptrs & 15) == 0) {
        const int warps = 8;
        const long long blocks = (vec_work + warps - 1) / warps;
        if (blocks > 2147483647LL) return SHARPI_BAD_ARGUMENT;
#define QKV_CASE(TO, P)                                                                     \
    do {                                                                                    \
        auto kern = qkv_post_vec_kernel<TO, P>;                                             \
        SHARPI_LAUNCH_PDL(kern, (unsigned)blocks, warps * 32, 0, stream, a);                \
    } while (0)
        if (out_dtype == SHARPI_F32) {
            if (d <= 128) QKV_CASE(float, 1); else if (d <= 256) QKV_CASE(float, 2); else QKV_CASE(float, 4);
        } else {
            if (d <= 128) QKV_CASE(bf16, 1); else if (d <= 256) QKV_CASE(bf16, 2); else QKV_CASE(bf16, 4);
        }
#undef QKV_CASE
        return SHARPI_OK;
    }
    const int warps = 4;
    const long long blocks = (work + warps - 1) / warps;
    if (blocks > 2147483647LL) return SHARPI_BAD_ARGUMENT;
    if (out_dtype == SHARPI_F32)
        qkv_post_kernel<float><<<(unsigned)blocks, warps * 32, 0, stream>>>(a);
    else if (out_dtype == SHARPI_BF16)
        qkv_post_kernel<bf16><<<(unsigned)blocks, warps * 32, 0, stream>>>(a);
    else
        return SHARPI_BAD_ARGUMENT;
    SHARPI_CHECK_LAUNCH();
    return SHARPI_OK;
}

// ---------------------------------------------------------------------------------------------------------
// The general form: heads padded to D elements whose keys use the first `dk` and whose values the first `dv`;
// an RMS norm with a weight on q and k over their dk elements BEFORE the rotation; a rotation of the first
// `rot` elements of q and k only (pairs (i, i + rot/2) or (2i, 2i+1) within those); and a rotation of every
// value by its own position over its first `vrot` elements with a frequency table of its own, so that the
// cache holds rotated values (the head's output is turned back by sharpi_rotate_heads).  One warp a (row, head).
struct QkvRotArgs {
    const float* qkv;        // [T, (nq + 2 nkv) * D]
    const int* positions;
    const int* row_req;
    const int* block_table;
    const float* q_norm_w;   // [dk] or null: no norm on q and k
    const float* k_norm_w;
    const float* inv_freq;   // [rot / 2] or null
    const float* inv_freq_v; // [vrot / 2] or null
    void* q_out;
    void* kv_base;
    int T, nq, nkv, D, dk, dv, rot, vrot;
    int max_blocks, page_size, pairing, write_kv;
    float eps;
};

// element i of a head after the rotation of its first `rot` elements by pos * inv_freq[pair]; val(i) gives the
// element before the rotation
template <typename F>
__device__ __forceinline__ float rotated_element(int i, int rot, int pairing, const float* inv_freq, float pos,
                                                 float sign, F val) {
    const float own = val(i);
    if (i >= rot || !inv_freq) return own;
    const int half = rot >> 1;
    int pair, other;
    bool is_first;
    if (pairing == ROPE_HALVES) {
        is_first = i < half;
        pair = is_first ? i : i - half;
        other = is_first ? i + half : i - half;
    } else {
        is_first = (i & 1) == 0;
        pair = i >> 1;
        other = is_first ? i + 1 : i - 1;
    }
    float sn, cs;
    sincosf(sign * pos * inv_freq[pair], &sn, &cs);
    const float o = val(other);
    return is_first ? own * cs - o * sn : own * cs + o * sn;
}

template <typename TO>
__global__ void __launch_bounds__(256) qkv_post_rot_kernel(QkvRotArgs a) {
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots = a.nq + 2 * a.nkv;
    const long long work = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (work >= (long long)a.T * slots) return;
    const int t = (int)(work / slots), slot = (int)(work % slots);
    const int D = a.D;
    const int pos = a.positions[t];
    const float* src = a.qkv + ((size_t)t * slots + slot) * D;
    const bool is_q = slot < a.nq;
    const bool is_k = !is_q && slot < a.nq + a.nkv;
    TO* dst;
    if (is_q) {
        dst = (TO*)a.q_out + ((size_t)t * a.nq + slot) * D;
    } else {
        if (!a.write_kv) return;
        const int head = is_k ? slot - a.nq : slot - a.nq - a.nkv;
        const int page = a.block_table[(size_t)a.row_req[t] * a.max_blocks + pos / a.page_size];
        if (page < 0) return;
        const size_t plane = (size_t)a.nkv * a.page_size * D;
        dst = (TO*)a.kv_base + ((size_t)page * 2 + (is_k ? 0 : 1)) * plane +
              ((size_t)head * a.page_size + (pos % a.page_size)) * D;
    }
    if (is_q || is_k) {
        const float* w = is_q ? a.q_norm_w : a.k_norm_w;
        float scale = 1.0f;
        if (w) {
            float ss = 0.0f;
            for (int i = lane; i < a.dk; i += 32) ss += src[i] * src[i];
            ss = warp_sum(ss);
            scale = 1.0f / sqrtf(ss / (float)a.dk + a.eps);
        }
        auto val = [&](int i) { return (w && i < a.dk) ? src[i] * scale * w[i] : src[i]; };
        for (int i = lane; i < D; i += 32)
            dst[i] = from_float<TO>(rotated_element(i, a.rot, a.pairing, a.inv_freq, (float)pos, 1.0f, val));
    } else {
        auto val = [&](int i) { return src[i]; };
        for (int i = lane; i < D; i += 32)
            dst[i] = from_float<TO>(rotated_element(i, a.vrot, a.pairing, a.inv_freq_v, (float)pos, 1.0f, val));
    }
}

SHARPI_API int sharpi_qkv_post_rot(const float* qkv, const int* positions, const int* row_req, const int* block_table,
                                   const float* q_norm_w, const float* k_norm_w, float eps, const float* inv_freq,
                                   int rot, const float* inv_freq_v, int vrot, int pairing, void* q_out, void* kv_base,
                                   int out_dtype, int T, int nq, int nkv, int D, int dk, int dv, int max_blocks,
                                   int page_size, int write_kv, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (nq <= 0 || nkv <= 0 || D <= 0 || dk <= 0 || dk > D || dv <= 0 || dv > D || page_size <= 0 || max_blocks <= 0)
        return SHARPI_BAD_ARGUMENT;
    if (rot < 0 || (rot & 1) || rot > dk || vrot < 0 || (vrot & 1) || vrot > dv) return SHARPI_BAD_ARGUMENT;
    if (pairing != ROPE_INTERLEAVED && pairing != ROPE_HALVES) return SHARPI_BAD_ARGUMENT;
    QkvRotArgs a;
    a.qkv = qkv; a.positions = positions; a.row_req = row_req; a.block_table = block_table;
    a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w; a.inv_freq = rot ? inv_freq : nullptr;
    a.inv_freq_v = vrot ? inv_freq_v : nullptr; a.q_out = q_out; a.kv_base = kv_base;
    a.T = T; a.nq = nq; a.nkv = nkv; a.D = D; a.dk = dk; a.dv = dv; a.rot = rot; a.vrot = vrot;
    a.max_blocks = max_blocks; a.page_size = page_size; a.pairing = pairing; a.write_kv = write_kv; a.eps = eps;
    const long long work = (long long)T * (nq + 2 * nkv);
    const long long blocks = (work + 7) / 8;
    if (blocks > 2147483647LL) return SHARPI_BAD_ARGUMENT;
    if (out_dtype == SHARPI_F32) SHARPI_LAUNCH_PDL(qkv_post_rot_kernel<float>, (unsigned)blocks, 256, 0, stream, a);
    else if (out_dtype == SHARPI_BF16) SHARPI_LAUNCH_PDL(qkv_post_rot_kernel<bf16>, (unsigned)blocks, 256, 0, stream, a);
    else return SHARPI_BAD_ARGUMENT;
    return SHARPI_OK;
}

// Every head of `in` [T, heads, D] turned by sign * position over its first `rot` elements (the rest copied):
// the inverse rotation of attention outputs whose values were cached rotated.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
rotate_heads_kernel(const TI* in, const int* positions, const float* __restrict__ inv_freq, TO* out, long long work,
                    int heads, int D, int rot, int pairing, float sign) {
    pdl_wait();
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= work) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(item / heads);
    const TI* src = in + (size_t)item * D;
    TO* dst = out + (size_t)item * D;
    const float pos = (float)positions[t];
    auto val = [&](int i) { return to_float(src[i]); };
    for (int i = lane; i < D; i += 32)
        dst[i] = from_float<TO>(rotated_element(i, rot, pairing, inv_freq, pos, sign, val));
}

SHARPI_API int sharpi_rotate_heads(const void* in, int in_dtype, const int* positions, const float* inv_freq, void* out,
                                   int out_dtype, int T, int heads, int D, int rot, int pairing, float sign,
                                   cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (heads <= 0 || D <= 0 || rot < 0 || (rot & 1) || rot > D) return SHARPI_BAD_ARGUMENT;
    if (pairing != ROPE_INTERLEAVED && pairing != ROPE_HALVES) return SHARPI_BAD_ARGUMENT;
    const long long work = (long long)T * heads;
    const unsigned blocks = (unsigned)((work + 7) / 8);
#define ROT_CASE(TI, TO)                                                                                         \
    SHARPI_LAUNCH_PDL((rotate_heads_kernel<TI, TO>), blocks, 256, 0, stream, (const TI*)in, positions, inv_freq, \
                      (TO*)out, work, heads, D, rot, pairing, sign)
    if (in_dtype == SHARPI_F32 && out_dtype == SHARPI_F32) ROT_CASE(float, float);
    else if (in_dtype == SHARPI_BF16 && out_dtype == SHARPI_BF16) ROT_CASE(bf16, bf16);
    else if (in_dtype == SHARPI_F32 && out_dtype == SHARPI_BF16) ROT_CASE(float, bf16);
    else return SHARPI_BAD_ARGUMENT;
#undef ROT_CASE
    return SHARPI_OK;
}

// ---------------------------------------------------------------------------------------
// The same pass for layers whose q/k norm runs over the WHOLE projection: q (all heads side by side) is divided by
// its root mean square and multiplied by a weight of that size, and so is k; no rotation.  Then the temperature
// factor on q, the store of q and the scatter of k and v into the pages.
//
//   qkv      float32 [T, ld]: q (nq * d) | k (nkv * d) | v (nkv * d); a layer that reads another layer's cache
//            brings q alone (`has_kv` = 0) and writes nothing.
//   wq, wk   float32 [nq * d], [nkv * d]; q_count / k_count: what the mean of squares divides by (fewer than the
//            row's elements when heads are padded with zeros).
//
// One block a row: the two sums of squares are formed by NORM_W_THREADS threads in a fixed order, so a row's
// numbers do not depend on the batch.  float32 throughout; q and the pages take the activation dtype.
// ---------------------------------------------------------------------------------------
constexpr int NORM_W_THREADS = 256;
static_assert(NORM_W_THREADS == 256, "the two-sum reduction below lays eight warps' sums side by side");

template <typename TO>
__global__ void __launch_bounds__(NORM_W_THREADS)
qkv_post_wide_kernel(const float* qkv, int ld, const int* positions, const int* row_req, const int* block_table,
                     const float* __restrict__ wq, const float* __restrict__ wk, float eps, int q_count, int k_count,
                     TO* q_out, TO* kv_base, int nq, int nkv, int d, int max_blocks, int page_size, float temp_coef,
                     float temp_every, int write_kv, int has_kv) {
    __shared__ float scratch[32];
    pdl_wait();
    const int t = blockIdx.x;
    const float* row = qkv + (size_t)t * ld;
    const int nQ = nq * d, nK = nkv * d;
    const int pos = positions[t];
    const bool store_kv = has_kv && write_kv;
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x; i < nQ; i += NORM_W_THREADS) sq += row[i] * row[i];
    if (store_kv)
        for (int i = threadIdx.x; i < nK; i += NORM_W_THREADS) sk += row[nQ + i] * row[nQ + i];
    // both sums through one pass of the block's tree (a fixed order: the block size never changes)
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { scratch[warp] = sq; scratch[8 + warp] = sk; }
        __syncthreads();
        sq = warp_sum(lane < NORM_W_THREADS / 32 ? scratch[lane] : 0.0f);
        sk = warp_sum(lane < NORM_W_THREADS / 32 ? scratch[8 + lane] : 0.0f);
    }
    float fq = 1.0f / sqrtf(sq / (float)q_count + eps);
    if (temp_every > 0.0f) fq *= 1.0f + temp_coef * log1pf(floorf(((float)pos + 1.0f) / temp_every));
    TO* qo = q_out + (size_t)t * nQ;
    for (int i = threadIdx.x; i < nQ; i += NORM_W_THREADS) qo[i] = from_float<TO>(row[i] * fq * wq[i]);
    if (!store_kv) return;
    const float fk = 1.0f / sqrtf(sk / (float)k_count + eps);
    const int page = block_table[(size_t)row_req[t] * max_blocks + pos / page_size];
    if (page < 0) return;   // the host checks before the launch that every written position has a page
    const size_t plane = (size_t)nkv * page_size * d;
    TO* kdst = kv_base + (size_t)page * 2 * plane + (size_t)(pos % page_size) * d;
    for (int i = threadIdx.x; i < nK; i += NORM_W_THREADS) {
        const int head = i / d, e = i - head * d;
        const size_t at = (size_t)head * page_size * d + e;
        kdst[at] = from_float<TO>(row[nQ + i] * fk * wk[i]);
        kdst[plane + at] = from_float<TO>(row[nQ + nK + i]);
    }
}

// The same with the row in registers: R pieces of four floats a thread, all loads issued before the first is used, so
// the kernel is one trip to memory (a decode step is one block a row waiting for its loads).  Needs sizes that are
// multiples of four (a piece lies within one head of q, k or v) and 16-byte aligned rows.  A thread adds its pieces'
// squares in ascending order and the block's tree is fixed, so a row's numbers depend on the row alone; which of the
// forms runs depends on the layer's sizes, never on the step.
template <typename TO, int R>
__global__ void __launch_bounds__(NORM_W_THREADS)
qkv_post_wide_regs_kernel(const float* qkv, int ld, const int* positions, const int* row_req, const int* block_table,
                          const float* __restrict__ wq, const float* __restrict__ wk, float eps, int q_count, int k_count,
                          TO* q_out, TO* kv_base, int nq, int nkv, int d, int max_blocks, int page_size, float temp_coef,
                          float temp_every, int write_kv, int has_kv) {
    __shared__ float scratch[32];
    pdl_wait();
    const int t = blockIdx.x;
    const float4* row = reinterpret_cast<const float4*>(qkv + (size_t)t * ld);
    const int nQ = nq * d, nK = nkv * d;
    const bool store_kv = has_kv && write_kv;
    const int pieces = (store_kv ? nQ + 2 * nK : nQ) / 4;
    float4 x[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = r * NORM_W_THREADS + threadIdx.x;
        x[r] = i < pieces ? row[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int pos = positions[t];
    float sq = 0.0f, sk = 0.0f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int e = 4 * (r * NORM_W_THREADS + threadIdx.x);
        const float ss = x[r].x * x[r].x + x[r].y * x[r].y + x[r].z * x[r].z + x[r].w * x[r].w;
        if (e < nQ) sq += ss;
        else if (e < nQ + nK) sk += ss;
    }
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { scratch[warp] = sq; scratch[8 + warp] = sk; }
        __syncthreads();
        sq = warp_sum(lane < NORM_W_THREADS / 32 ? scratch[lane] : 0.0f);
        sk = warp_sum(lane < NORM_W_THREADS / 32 ? scratch[8 + lane] : 0.0f);
    }
    float fq = 1.0f / sqrtf(sq / (float)q_count + eps);
    if (temp_every > 0.0f) fq *= 1.0f + temp_coef * log1pf(floorf(((float)pos + 1.0f) / temp_every));
    const float fk = store_kv ? 1.0f / sqrtf(sk / (float)k_count + eps) : 0.0f;
    int page = -1;
    if (store_kv) page = block_table[(size_t)row_req[t] * max_blocks + pos / page_size];
    const size_t plane = (size_t)nkv * page_size * d;
    TO* kdst = kv_base + (page < 0 ? 0 : (size_t)page * 2 * plane + (size_t)(pos % page_size) * d);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int e = 4 * (r * NORM_W_THREADS + threadIdx.x);
        if (e < nQ) {
            const float4 w = *reinterpret_cast<const float4*>(wq + e);
            store4<TO>(q_out + (size_t)t * nQ + e,
                       make_float4(x[r].x * fq * w.x, x[r].y * fq * w.y, x[r].z * fq * w.z, x[r].w * fq * w.w));
        } else if (page >= 0 && e < nQ + 2 * nK) {      // the host checks that every written position has a page
            const bool is_k = e < nQ + nK;
            const int i = e - nQ - (is_k ? 0 : nK);
            const int head = i / d;
            TO* dst = kdst + (is_k ? 0 : plane) + (size_t)head * page_size * d + (i - head * d);
            if (is_k) {
                const float4 w = *reinterpret_cast<const float4*>(wk + i);
                store4<TO>(dst, make_float4(x[r].x * fk * w.x, x[r].y * fk * w.y, x[r].z * fk * w.z, x[r].w * fk * w.w));
            } else {
                store4<TO>(dst, x[r]);
            }
        }
    }
}

template <typename TO>
static int launch_wide(const float* qkv, int ld, const int* positions, const int* row_req, const int* block_table,
                       const float* wq, const float* wk, float eps, int q_count, int k_count, TO* q_out, TO* kv_base, int T,
                       int nq, int nkv, int d, int max_blocks, int page_size, float temp_coef, float temp_every,
                       int write_kv, int has_kv, cudaStream_t stream) {
    const int floats = (has_kv && write_kv) ? (nq + 2 * nkv) * d : nq * d;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                           reinterpret_cast<uintptr_t>(kv_base) | reinterpret_cast<uintptr_t>(wq) |
                           reinterpret_cast<uintptr_t>(wk);
    const bool pieces = d % 4 == 0 && ld % 4 == 0 && (ptrs & 15) == 0 && floats <= 8 * 4 * NORM_W_THREADS;
#define WIDE_ARGS qkv, ld, positions, row_req, block_table, wq, wk, eps, q_count, k_count, q_out, kv_base, nq, nkv, d, \
                  max_blocks, page_size, temp_coef, temp_every, write_kv, has_kv
    if (pieces && floats <= 2 * 4 * NORM_W_THREADS)
        SHARPI_LAUNCH_PDL((qkv_post_wide_regs_kernel<TO, 2>), T, NORM_W_THREADS, 0, stream, WIDE_ARGS);
    else if (pieces && floats <= 4 * 4 * NORM_W_THREADS)
        SHARPI_LAUNCH_PDL((qkv_post_wide_regs_kernel<TO, 4>), T, NORM_W_THREADS, 0, stream, WIDE_ARGS);
    else if (pieces)
        SHARPI_LAUNCH_PDL((qkv_post_wide_regs_kernel<TO, 8>), T, NORM_W_THREADS, 0, stream, WIDE_ARGS);
    else
        SHARPI_LAUNCH_PDL(qkv_post_wide_kernel<TO>, T, NORM_W_THREADS, 0, stream, WIDE_ARGS);
#undef WIDE_ARGS
    return SHARPI_OK;
}

SHARPI_API int sharpi_qkv_post_wide(const float* qkv, int ld, const int* positions, const int* row_req,
                                    const int* block_table, const float* wq, const float* wk, float eps, int q_count,
                                    int k_count, void* q_out, void* kv_base, int out_dtype, int T, int nq, int nkv,
                                    int d, int max_blocks, int page_size, float temp_coef, float temp_every,
                                    int write_kv, int has_kv, cudaStream_t stream) {
    if (T <= 0) return SHARPI_OK;
    if (nq <= 0 || nkv <= 0 || d <= 0 || page_size <= 0 || max_blocks <= 0 || !wq || q_count <= 0) return SHARPI_BAD_ARGUMENT;
    if (has_kv && (!wk || k_count <= 0 || ld < (nq + 2 * nkv) * d)) return SHARPI_BAD_ARGUMENT;
    if (ld < nq * d) return SHARPI_BAD_ARGUMENT;
    if (out_dtype == SHARPI_F32)
        return launch_wide<float>(qkv, ld, positions, row_req, block_table, wq, wk, eps, q_count, k_count, (float*)q_out,
                                  (float*)kv_base, T, nq, nkv, d, max_blocks, page_size, temp_coef, temp_every, write_kv,
                                  has_kv, stream);
    if (out_dtype == SHARPI_BF16)
        return launch_wide<bf16>(qkv, ld, positions, row_req, block_table, wq, wk, eps, q_count, k_count, (bf16*)q_out,
                                 (bf16*)kv_base, T, nq, nkv, d, max_blocks, page_size, temp_coef, temp_every, write_kv,
                                 has_kv, stream);
    return SHARPI_BAD_ARGUMENT;
}
