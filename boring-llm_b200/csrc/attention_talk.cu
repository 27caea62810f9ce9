// Paged attention whose heads' weights are mixed AFTER the softmax ("talking heads"), over keys limited to the query's
// own chunk of positions:
//   score_g(i, j) = q_g(i) . k_kv(g)(j) * scale * head_scale[g],  j in [lo(i), i],  lo(i) = i - i % chunk  (chunk 0: lo = 0;
//                   window > 0: lo = max(lo, i - window + 1))
//   W_g = softmax_j(score_g),   W'_h = sum_g talk[h, g] W_g,   out_h(i) = sum_j W'_h(i, j) v_kv(h)(j)
// Since the mix is linear, out_h = sum_g talk[h, g] A[g, kv(h)] with A[g, c](i) = sum_j W_g(i, j) v_c(j): every query
// head's softmax is applied to the values of EVERY key/value head in one pass over the keys (online softmax, nothing of
// size keys x keys is stored), and a small kernel mixes the heads. Chunks are counted from position 0 of the sequence.
// This file holds the plain kernel (one warp per (token, head), any dtype: the 32-bit path and the twin of the
// tensor-core kernels) and the mix. On tensor cores the same is bl_attention_prefill_talk / bl_attention_decode_talk in
// attention_mma.cu: its two shapes with a first visible key per row, a scale per head, and the values of a chosen head.
#include "common.cuh"
#include "api.h"

namespace {

constexpr int MAX_DH = 256;
constexpr int WARPS = 4;
constexpr int ACC = 16;                                // accumulators a lane holds: value heads in a pass x ceil(dv / 32)

__device__ __forceinline__ int first_visible(int pos, int chunk, int window) {
    int lo = chunk > 0 ? pos - pos % chunk : 0;
    if (window > 0) lo = max(lo, pos - window + 1);
    return lo;
}

template <typename TT, int NV>
__global__ void __launch_bounds__(WARPS * 32)
attention_talk_plain_kernel(const TT* __restrict__ q, const TT* __restrict__ kc, const TT* __restrict__ vc,
                            const int* __restrict__ tok_req, const int* __restrict__ cu_q, const int* __restrict__ ctx_len,
                            const int* __restrict__ block_table, int max_pages, float* __restrict__ A, int T, int H, int KV,
                            int dh, int dv, int page_size, int chunk, int window, float scale,
                            const void* __restrict__ head_scale, int hs_dtype) {
    constexpr int CG = ACC / NV;                       // value heads in a pass
    __shared__ float qs[WARPS][MAX_DH];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int item = blockIdx.x * WARPS + warp;
    if (item >= T * H) return;
    const int c0 = blockIdx.y * CG;
    const int t = item / H, g = item % H;
    const int r = tok_req[t];
    const int q_len = cu_q[r + 1] - cu_q[r];
    const int pos = ctx_len[r] - q_len + (t - cu_q[r]);
    const int kvh = g / (H / KV);
    const int lo = first_visible(pos, chunk, window);
    const float sc = scale * (head_scale ? bl_load_any(head_scale, hs_dtype, g) : 1.f);
    const TT* qrow = q + ((size_t)t * H + g) * dh;
    for (int d = lane; d < dh; d += 32) qs[warp][d] = bl_load(qrow + d);
    __syncwarp();
    const int* bt = block_table + (size_t)r * max_pages;
    const size_t head_off = (size_t)kvh * page_size * dh;
    const size_t page_stride = (size_t)KV * page_size * dh, v_page_stride = (size_t)KV * page_size * dv;
    float m = -INFINITY, l = 0.f;
    float acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
    for (int base = lo; base <= pos; base += 32) {
        const int j = base + lane;
        const bool valid = j <= pos;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / page_size];
            const TT* krow = kc + (size_t)page * page_stride + head_off + (size_t)(j % page_size) * dh;
            float dot = 0.f;
            for (int d = 0; d < dh; ++d) dot = fmaf(qs[warp][d], bl_load(krow + d), dot);
            s = dot * sc;
        }
        const float m_new = fmaxf(m, bl_warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);
        l = l * alpha + bl_warp_sum(p);
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] *= alpha;
        const int n = min(32, pos - base + 1);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int key = base + jj;
            const TT* vpage = vc + (size_t)bt[key / page_size] * v_page_stride + (size_t)(key % page_size) * dv;
#pragma unroll
            for (int cl = 0; cl < CG; ++cl) {
                if (c0 + cl < KV) {
                    const TT* vrow = vpage + (size_t)(c0 + cl) * page_size * dv;
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        const int d = lane + 32 * i;
                        if (d < dv) acc[cl * NV + i] = fmaf(pj, bl_load(vrow + d), acc[cl * NV + i]);
                    }
                }
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int cl = 0; cl < CG; ++cl) {
        if (c0 + cl < KV) {
            float* dst = A + (((size_t)t * H + g) * KV + c0 + cl) * dv;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) dst[d] = acc[cl * NV + i] * inv;
            }
        }
    }
}

// out[t, h, :] = sum_g talk[h, g] * A[t, g, kv(h), :], g ascending; one block per token, the mix matrix in shared memory
// (fetched before the dependent-launch wait: it is a weight), a thread per pair of channels where dv is even.
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void store2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float a, float b) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b); }

template <typename TA, typename TT>
__global__ void __launch_bounds__(128)
talk_mix_kernel(const TA* __restrict__ A, const void* __restrict__ talk, int talk_dtype, TT* __restrict__ out, int H, int KV, int dv) {
    bl_pdl_trigger();
    extern __shared__ float tk[];                      // [H, H]
    for (int i = threadIdx.x; i < H * H; i += 128) tk[i] = bl_load_any(talk, talk_dtype, i);
    bl_pdl_wait();
    __syncthreads();
    const int t = blockIdx.x;
    const int rep = H / KV;
    const size_t g_step = (size_t)KV * dv;             // from head g to head g + 1 in A[t]
    const TA* At = A + (size_t)t * H * g_step;
    if ((dv & 1) == 0) {
        const int half = dv >> 1;
        for (int e = threadIdx.x; e < H * half; e += 128) {
            const int h = e / half, d = (e - h * half) * 2;
            const TA* src = At + (size_t)(h / rep) * dv + d;
            const float* row = tk + h * H;
            float a0 = 0.f, a1 = 0.f;
            for (int g = 0; g < H; ++g) {
                const float2 v = load2(src + g * g_step);
                a0 = fmaf(row[g], v.x, a0);
                a1 = fmaf(row[g], v.y, a1);
            }
            store2(out + (size_t)t * H * dv + (size_t)h * dv + d, a0, a1);
        }
        return;
    }
    for (int e = threadIdx.x; e < H * dv; e += 128) {
        const int h = e / dv, d = e % dv;
        const TA* src = At + (size_t)(h / rep) * dv + d;
        float acc = 0.f;
        for (int g = 0; g < H; ++g) acc = fmaf(tk[h * H + g], bl_load(src + g * g_step), acc);
        bl_store(out + (size_t)t * H * dv + e, acc);
    }
}

}  // namespace

extern "C" int bl_attention_talk_plain(const void* q, const void* k_cache, const void* v_cache, int dtype, const int* tok_req,
                                       const int* cu_q, const int* ctx_len, const int* block_table, int max_pages, float* A,
                                       int T, int H, int KV, int dh, int dv, int page_size, int chunk, int window, float scale,
                                       const void* head_scale, int hs_dtype, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV != 0) BL_FAIL("bl_attention_talk_plain: %d heads cannot share %d key/value heads", H, KV);
    if (dh <= 0 || dh > MAX_DH || dv <= 0 || dv > MAX_DH) BL_FAIL("bl_attention_talk_plain: head sizes %d / %d are outside 1..%d", dh, dv, MAX_DH);
    if (page_size <= 0 || max_pages <= 0 || chunk < 0 || window < 0) BL_FAIL("bl_attention_talk_plain: bad page size, table width, chunk or window");
    cudaStream_t s = (cudaStream_t)stream;
    const int nv = (dv + 31) / 32;
    const int NV = nv <= 1 ? 1 : nv <= 2 ? 2 : nv <= 4 ? 4 : 8;
    const int cg = ACC / NV;
    const dim3 grid((T * H + WARPS - 1) / WARPS, (KV + cg - 1) / cg);
#define BL_GO(TT, NV_) attention_talk_plain_kernel<TT, NV_><<<grid, WARPS * 32, 0, s>>>((const TT*)q, (const TT*)k_cache, (const TT*)v_cache, \
        tok_req, cu_q, ctx_len, block_table, max_pages, A, T, H, KV, dh, dv, page_size, chunk, window, scale, head_scale, hs_dtype)
#define BL_GO_NV(TT) do { if (NV == 1) BL_GO(TT, 1); else if (NV == 2) BL_GO(TT, 2); else if (NV == 4) BL_GO(TT, 4); else BL_GO(TT, 8); } while (0)
    if (dtype == BL_F32) BL_GO_NV(float);
    else if (dtype == BL_BF16) BL_GO_NV(__nv_bfloat16);
    else BL_FAIL("bl_attention_talk_plain: unknown dtype %d", dtype);
#undef BL_GO_NV
#undef BL_GO
    BL_CHECK_LAUNCH("bl_attention_talk_plain");
    return 0;
}

extern "C" int bl_talk_mix(const void* A, int a_dtype, const void* talk, int talk_dtype, void* out, int out_dtype, int T, int H, int KV,
                           int dv, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || KV <= 0 || H % KV != 0 || dv <= 0) BL_FAIL("bl_talk_mix: bad sizes H=%d KV=%d dv=%d", H, KV, dv);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)H * H * sizeof(float);
    if (smem > 48 * 1024) BL_FAIL("bl_talk_mix: %d heads are too many for shared memory", H);
#define BL_GO(TA, TT) BL_CUDA(bl_launch_dependent(talk_mix_kernel<TA, TT>, dim3(T), dim3(128), smem, s, (const TA*)A, talk, talk_dtype, (TT*)out, H, KV, dv))
    if (a_dtype == BL_F32 && out_dtype == BL_F32) BL_GO(float, float);
    else if (a_dtype == BL_F32 && out_dtype == BL_BF16) BL_GO(float, __nv_bfloat16);
    else if (a_dtype == BL_BF16 && out_dtype == BL_BF16) BL_GO(__nv_bfloat16, __nv_bfloat16);
    else BL_FAIL("bl_talk_mix: unsupported dtypes %d -> %d", a_dtype, out_dtype);
#undef BL_GO
    BL_CHECK_LAUNCH("bl_talk_mix");
    return 0;
}
