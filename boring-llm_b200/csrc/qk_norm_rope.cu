// Between the joined q/k/v product and the paged cache, for attention whose queries and keys are normed over the WHOLE
// projection (all heads of a token at once, before they are split) and whose values may have another head size than
// its keys: RMS norm of the token's q row and of its k row with plain weights, rotation of the first 2 * rot_half
// dimensions of every head (pairs (2j, 2j + 1) or (j, j + rot_half)), q out, k and v into the pages of the token's
// request. Statistics, angles and the rotation are 32-bit; angle = float(position) * inv_freq[j].
#include "common.cuh"
#include "api.h"

namespace {

constexpr int THREADS = 128;

__device__ __forceinline__ float block_sum(float v, float* part) {
    v = bl_warp_sum(v);
    __syncthreads();                                   // part may still be read from the call before
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    return (part[0] + part[1]) + (part[2] + part[3]);
}

template <typename TT>
__global__ void __launch_bounds__(THREADS)
qk_norm_rope_write_kernel(const float* proj, int ld, int off_k, int off_v, const void* __restrict__ qw, int qw_dtype,
                          const void* __restrict__ kw, int kw_dtype, float eps, const int* __restrict__ positions,
                          const int* __restrict__ tok_req, const int* __restrict__ block_table, int max_pages,
                          const float* __restrict__ inv_freq, int rot_half, int pair_layout, TT* __restrict__ q_out,
                          TT* __restrict__ k_cache, TT* __restrict__ v_cache, int H, int KV, int dk, int dv, int page_size,
                          int per_head, const float* __restrict__ q_head_scale) {
    bl_pdl_trigger();
    bl_pdl_wait();
    extern __shared__ float cs[];                      // cos [rot_half], sin [rot_half], then (per_head) 1 / rms of each of the H + KV heads
    __shared__ float part[4];
    const int t = blockIdx.x;
    const float* row = proj + (size_t)t * ld;
    const int pos = positions[t];
    for (int j = threadIdx.x; j < rot_half; j += THREADS) {
        const float a = (float)pos * inv_freq[j];
        cs[j] = cosf(a);
        cs[rot_half + j] = sinf(a);
    }
    float inv_q = 1.f, inv_k = 1.f;
    float* inv_head = cs + 2 * rot_half;
    if (per_head) {                                    // a norm over each head's dk values; the weights [dk] are shared by the heads
        const int lane = threadIdx.x & 31;
        for (int hh = threadIdx.x >> 5; hh < H + KV; hh += THREADS / 32) {
            const float* hr = row + (hh < H ? hh * dk : off_k + (hh - H) * dk);
            float s = 0.f;
            for (int i = lane; i < dk; i += 32) s += hr[i] * hr[i];
            s = bl_warp_sum(s);
            if (lane == 0) inv_head[hh] = ((hh < H ? qw : kw) != nullptr) ? 1.0f / sqrtf(s / (float)dk + eps) : 1.f;
        }
    } else if (qw) {
        float s = 0.f;
        for (int i = threadIdx.x; i < H * dk; i += THREADS) s += row[i] * row[i];
        inv_q = 1.0f / sqrtf(block_sum(s, part) / (float)(H * dk) + eps);
    }
    if (kw && !per_head) {
        float s = 0.f;
        for (int i = threadIdx.x; i < KV * dk; i += THREADS) s += row[off_k + i] * row[off_k + i];
        inv_k = 1.0f / sqrtf(block_sum(s, part) / (float)(KV * dk) + eps);
    }
    __syncthreads();
    const int r = tok_req[t];
    const int page = k_cache || v_cache ? block_table[(size_t)r * max_pages + pos / page_size] : 0;
    const int in_page = pos % page_size;
    const int n_rot = 2 * rot_half;
    // heads 0 .. H - 1 are q's, H .. H + KV - 1 are k's
    for (int e = threadIdx.x; e < (H + KV) * dk; e += THREADS) {
        const int hh = e / dk, d = e % dk;
        const bool is_q = hh < H;
        const int col = is_q ? hh * dk : off_k + (hh - H) * dk;        // the head's first column in the row
        const int wcol = per_head ? 0 : (is_q ? hh * dk : (hh - H) * dk);
        const void* w = is_q ? qw : kw;
        const int wd = is_q ? qw_dtype : kw_dtype;
        const float inv = per_head ? inv_head[hh] : (is_q ? inv_q : inv_k);
        auto normed = [&](int dd) { return row[col + dd] * inv * (w ? bl_load_any(w, wd, wcol + dd) : 1.f); };
        float val;
        if (d < n_rot) {
            int j, other;
            bool first;
            if (pair_layout == BL_PAIRS_INTERLEAVED) { j = d >> 1; first = (d & 1) == 0; other = first ? d + 1 : d - 1; }
            else { first = d < rot_half; j = first ? d : d - rot_half; other = first ? d + rot_half : d - rot_half; }
            const float c = cs[j], s = cs[rot_half + j];
            const float me = normed(d), ot = normed(other);
            val = first ? me * c - ot * s : me * c + ot * s;
        } else {
            val = normed(d);
        }
        if (is_q) {
            bl_store(q_out + (size_t)t * H * dk + e, q_head_scale ? val * q_head_scale[hh] : val);
        } else if (k_cache) {
            bl_store(k_cache + (((size_t)page * KV + (hh - H)) * page_size + in_page) * dk + d, val);
        }
    }
    if (v_cache) {
        for (int e = threadIdx.x; e < KV * dv; e += THREADS) {
            const int g = e / dv, d = e % dv;
            bl_store(v_cache + (((size_t)page * KV + g) * page_size + in_page) * dv + d, row[off_v + e]);
        }
    }
}

}  // namespace

extern "C" int bl_qk_norm_rope_write(const float* proj, int ld, int off_k, int off_v, const void* q_norm_w, int qw_dtype,
                                     const void* k_norm_w, int kw_dtype, float eps, const int* positions, const int* tok_req,
                                     const int* block_table, int max_pages, const float* inv_freq, int rot_half,
                                     int pair_layout, void* q_out, void* k_cache, void* v_cache, int dtype, int T, int H,
                                     int KV, int dk, int dv, int page_size, void* stream) {
    return bl_qk_norm_rope_write_scope(proj, ld, off_k, off_v, q_norm_w, qw_dtype, k_norm_w, kw_dtype, eps, 0, positions, tok_req,
                                       block_table, max_pages, inv_freq, rot_half, pair_layout, q_out, k_cache, v_cache, dtype, T, H,
                                       KV, dk, dv, page_size, nullptr, stream);
}

extern "C" int bl_qk_norm_rope_write_scope(const float* proj, int ld, int off_k, int off_v, const void* q_norm_w, int qw_dtype,
                                           const void* k_norm_w, int kw_dtype, float eps, int per_head, const int* positions,
                                           const int* tok_req, const int* block_table, int max_pages, const float* inv_freq,
                                           int rot_half, int pair_layout, void* q_out, void* k_cache, void* v_cache, int dtype, int T,
                                           int H, int KV, int dk, int dv, int page_size, const float* q_head_scale, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || KV <= 0 || dk <= 0 || dv <= 0 || rot_half < 0 || 2 * rot_half > dk || page_size <= 0)
        BL_FAIL("bl_qk_norm_rope_write: bad sizes H=%d KV=%d dk=%d dv=%d rotated pairs=%d page=%d", H, KV, dk, dv, rot_half, page_size);
    if (ld < off_v + KV * dv || off_k < H * dk || off_v < off_k + KV * dk)
        BL_FAIL("bl_qk_norm_rope_write: columns q, k (%d), v (%d) do not fit rows of %d", off_k, off_v, ld);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(2 * rot_half + 1 + (per_head ? H + KV : 0)) * sizeof(float);
#define BL_GO(TT) BL_CUDA(bl_launch_dependent(qk_norm_rope_write_kernel<TT>, dim3(T), dim3(THREADS), smem, s, proj, ld, off_k, off_v, \
        q_norm_w, qw_dtype, k_norm_w, kw_dtype, eps, positions, tok_req, block_table, max_pages, inv_freq, rot_half, pair_layout, \
        (TT*)q_out, (TT*)k_cache, (TT*)v_cache, H, KV, dk, dv, page_size, per_head, q_head_scale))
    if (dtype == BL_F32) BL_GO(float);
    else if (dtype == BL_BF16) BL_GO(__nv_bfloat16);
    else BL_FAIL("bl_qk_norm_rope_write: unknown dtype %d", dtype);
#undef BL_GO
    BL_CHECK_LAUNCH("bl_qk_norm_rope_write");
    return 0;
}
