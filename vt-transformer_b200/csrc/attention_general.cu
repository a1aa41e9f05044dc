// The general attention: values of another size than keys, a rotation of the first dimensions of a head only with
// the angle formed where it is used, q and k divided by their root mean square after the rotation, and a mask of
// chunks beside the causal one and the window.
//
// Two kernels.  `attention_prepare` (one block a token, one warp a head): rotation of pairs (i, i + half) by
// position * frequency[i] (a 32-bit product, precise sine and cosine), the norm over the head in 32-bit, q written
// back in place, k and v stored into their pages.  `attention_general` (one warp for a (token, head)): the visible
// keys one after the other in the order of their positions with a running maximum and sum in 32-bit, as in the plain
// attention kernel, so that a token's result depends on its own keys only.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {
constexpr int kMaxPerLane = 8;       // head sizes up to 256
constexpr int kPrepareWarps = 4;
}

template <typename T>
__global__ void __launch_bounds__(32 * kPrepareWarps)
attention_prepare_kernel(T* __restrict__ y, int stride, int q_col, int k_col, int v_col, const int* __restrict__ positions,
                         const int* __restrict__ token_seq, const float* __restrict__ freq, int half, float norm_eps,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ block_table,
                         int table_stride, int n_seqs, int n_pages, int heads, int kv_heads, int dim, int v_dim,
                         int page_size, int store, int* status) {
    __shared__ float head[kPrepareWarps][32 * kMaxPerLane];
    pdl_launch();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int seq = token_seq[t];
    const bool seq_ok = seq >= 0 && seq < n_seqs;
    const int pos = seq_ok ? positions[t] : 0;
    const int page = (store && seq_ok && pos >= 0) ? block_table[(size_t)seq * table_stride + pos / page_size] : 0;
    pdl_wait();
    if (seq < 0) return;   // padding
    if (!seq_ok) {
        if (threadIdx.x == 0) set_status(status, kStatusBadSequence, seq);
        return;
    }
    if (pos < 0) {
        if (threadIdx.x == 0) set_status(status, kStatusBadPosition, pos);
        return;
    }
    if (store && (page < 0 || page >= n_pages)) {
        if (threadIdx.x == 0) set_status(status, kStatusBadPage, page);
        store = 0;
    }
    T* row = y + (size_t)t * stride;
    const int slot = pos % page_size;
    const int units = heads + (store ? kv_heads : 0);
    float* hv = head[warp];
    for (int u = warp; u < units; u += kPrepareWarps) {
        const bool is_q = u < heads;
        T* src = is_q ? row + q_col + u * dim : row + k_col + (u - heads) * dim;
        for (int i = lane; i < dim; i += 32) hv[i] = to_float(src[i]);
        __syncwarp();
        float x[kMaxPerLane];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) {
            const int i = lane + 32 * r;
            float v = 0.f;
            if (i < dim) {
                v = hv[i];
                if (i < 2 * half) {
                    const int f = i < half ? i : i - half;
                    const float angle = (float)pos * freq[f];
                    float sn, cs;
                    sincosf(angle, &sn, &cs);
                    v = i < half ? v * cs - hv[i + half] * sn : v * cs + hv[i - half] * sn;
                }
            }
            x[r] = v;
            ss = fmaf(v, v, ss);
        }
        float scale = 1.f;
        if (norm_eps >= 0.f) scale = rsqrtf(warp_sum(ss) / (float)dim + norm_eps);
        T* dst = is_q ? src : k_cache + (((size_t)page * kv_heads + (u - heads)) * page_size + slot) * dim;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) {
            const int i = lane + 32 * r;
            if (i < dim) dst[i] = from_float<T>(x[r] * scale);
        }
        __syncwarp();
    }
    if (!store) return;
    for (int e = threadIdx.x; e < kv_heads * v_dim; e += blockDim.x) {
        const int h = e / v_dim, i = e % v_dim;
        v_cache[(((size_t)page * kv_heads + h) * page_size + slot) * v_dim + i] = row[v_col + e];
    }
}

cudaError_t launch_attention_prepare(int dtype, void* y, int stride, int q_col, int k_col, int v_col, const int* positions,
                                     const int* token_seq, const float* freq, int half, float norm_eps, void* k_cache,
                                     void* v_cache, const int* block_table, int table_stride, int n_seqs, int n_pages,
                                     int n_tokens, int heads, int kv_heads, int dim, int v_dim, int page_size, int store,
                                     int* status, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (dim > 32 * kMaxPerLane || 2 * half > dim) return cudaErrorInvalidValue;
    if (dtype == kBF16)
        return launch(attention_prepare_kernel<__nv_bfloat16>, n_tokens, 32 * kPrepareWarps, 0, stream, (__nv_bfloat16*)y, stride,
                      q_col, k_col, v_col, positions, token_seq, freq, half, norm_eps, (__nv_bfloat16*)k_cache,
                      (__nv_bfloat16*)v_cache, block_table, table_stride, n_seqs, n_pages, heads, kv_heads, dim, v_dim,
                      page_size, store, status);
    return launch(attention_prepare_kernel<float>, n_tokens, 32 * kPrepareWarps, 0, stream, (float*)y, stride, q_col, k_col,
                  v_col, positions, token_seq, freq, half, norm_eps, (float*)k_cache, (float*)v_cache, block_table,
                  table_stride, n_seqs, n_pages, heads, kv_heads, dim, v_dim, page_size, store, status);
}

// One warp for a (token, head).  The visible keys are taken 32 at a time, a lane a key: the lane forms its key's whole
// score from q in shared memory (no exchange between lanes for a score), the block's maximum and sum are found once,
// and the block's values are added with a lane owning dimensions i, i + 32, ... of the result.  The blocks start at the
// first visible key, which depends on the token's position alone, so a token's result does not depend on the step.
template <typename T, bool Vec>
__global__ void __launch_bounds__(128)
attention_general_kernel(const T* __restrict__ y, int stride, int q_col, T* __restrict__ out, int out_stride, int out_col,
                         float out_scale, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                         const int* __restrict__ block_table, int table_stride, int n_seqs, int n_pages, int n_tokens,
                         int heads, int kv_heads, int dim, int v_dim, int page_size, int window, int chunk, float scale,
                         int* status) {
    __shared__ __align__(16) float qs[4][32 * kMaxPerLane];
    pdl_launch();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (pair >= (long long)n_tokens * heads) return;
    const int t = (int)(pair / heads), h = (int)(pair % heads);
    const int seq = token_seq[t];
    T* o = out + (size_t)t * out_stride + out_col + (size_t)h * v_dim;
    if (seq < 0) {   // padding
        for (int i = lane; i < v_dim; i += 32) o[i] = from_float<T>(0.f);
        return;
    }
    if (seq >= n_seqs) {
        if (lane == 0) set_status(status, kStatusBadSequence, seq);
        return;
    }
    const int pos = positions[t];
    const int kvh = h / (heads / kv_heads);
    const int* table = block_table + (size_t)seq * table_stride;
    float* q = qs[warp];
    const T* qp = y + (size_t)t * stride + q_col + (size_t)h * dim;
    for (int i = lane; i < dim; i += 32) q[i] = to_float(qp[i]) * scale;
    __syncwarp();

    float acc[kMaxPerLane];
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) acc[r] = 0.f;
    float mx = -INFINITY, sum = 0.f;
    int first = (window > 0) ? max(0, pos - window + 1) : 0;
    if (chunk > 0) first = max(first, (pos / chunk) * chunk);      // chunks are counted from position 0 of the sequence
    for (int j0 = first; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        bool live = j <= pos;
        int at = 0;                                                // the key's row in the pages
        if (live) {
            const int page = table[j / page_size];
            if (page < 0 || page >= n_pages) {
                set_status(status, kStatusBadPage, page);
                live = false;
            } else {
                at = (page * kv_heads + kvh) * page_size + (j % page_size);
            }
        }
        float s = -INFINITY;
        if (live) {
            const T* kp = k_cache + (size_t)at * dim;
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            if (Vec) {
                for (int i = 0; i < dim; i += 8) {
                    float k8[8];
                    Vec8<T>::load(kp + i, k8);
                    const float4 qa = *reinterpret_cast<const float4*>(q + i), qb = *reinterpret_cast<const float4*>(q + i + 4);
                    part[0] = fmaf(qa.x, k8[0], part[0]); part[1] = fmaf(qa.y, k8[1], part[1]);
                    part[2] = fmaf(qa.z, k8[2], part[2]); part[3] = fmaf(qa.w, k8[3], part[3]);
                    part[0] = fmaf(qb.x, k8[4], part[0]); part[1] = fmaf(qb.y, k8[5], part[1]);
                    part[2] = fmaf(qb.z, k8[6], part[2]); part[3] = fmaf(qb.w, k8[7], part[3]);
                }
            } else {
                for (int i = 0; i < dim; ++i) part[i & 3] = fmaf(q[i], to_float(kp[i]), part[i & 3]);
            }
            s = (part[0] + part[1]) + (part[2] + part[3]);
        }
        const float new_mx = fmaxf(mx, warp_max(s));              // the first block holds the token's own key: finite
        const float corr = expf(mx - new_mx);                      // 0 at the first block (mx = -inf)
        const float p = live ? expf(s - new_mx) : 0.f;
        sum = sum * corr + warp_sum(p);
        mx = new_mx;
#pragma unroll
        for (int r = 0; r < kMaxPerLane; ++r) acc[r] *= corr;
        const int n = min(32, pos - j0 + 1);
        for (int jj = 0; jj < n; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int aj = __shfl_sync(0xffffffffu, at, jj);
            const T* vp = v_cache + (size_t)aj * v_dim;
#pragma unroll
            for (int r = 0; r < kMaxPerLane; ++r) {
                const int i = lane + 32 * r;
                if (i < v_dim) acc[r] = fmaf(pj, to_float(vp[i]), acc[r]);
            }
        }
    }
    const float inv = sum > 0.f ? out_scale / sum : 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPerLane; ++r) {
        const int i = lane + 32 * r;
        if (i < v_dim) o[i] = from_float<T>(acc[r] * inv);
    }
}

template <typename T>
static cudaError_t launch_attention_general_t(const T* y, int stride, int q_col, T* out, int out_stride, int out_col, float out_scale,
                                              const T* k_cache, const T* v_cache, const int* positions, const int* token_seq,
                                              const int* block_table, int table_stride, int n_seqs, int n_pages, int n_tokens,
                                              int heads, int kv_heads, int dim, int v_dim, int page_size, int window, int chunk,
                                              float scale, int* status, cudaStream_t stream) {
    const long long pairs = (long long)n_tokens * heads;
    const int blocks = (int)((pairs + 3) / 4);
    // a key's row is read in 16-byte pieces where every row starts on such a boundary
    const bool vec = dim % 8 == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0;
    auto kernel = vec ? attention_general_kernel<T, true> : attention_general_kernel<T, false>;
    return launch(kernel, blocks, 128, 0, stream, y, stride, q_col, out, out_stride, out_col, out_scale, k_cache, v_cache, positions,
                  token_seq, block_table, table_stride, n_seqs, n_pages, n_tokens, heads, kv_heads, dim, v_dim, page_size, window,
                  chunk, scale, status);
}

cudaError_t launch_attention_general(int dtype, const void* y, int stride, int q_col, void* out, int out_stride, int out_col,
                                     float out_scale, const void* k_cache, const void* v_cache, const int* positions,
                                     const int* token_seq, const int* block_table, int table_stride, int n_seqs, int n_pages,
                                     int n_tokens, int heads, int kv_heads, int dim, int v_dim, int page_size, int window,
                                     int chunk, float scale, int* status, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (dim > 32 * kMaxPerLane || v_dim > 32 * kMaxPerLane) return cudaErrorInvalidValue;
    if (dtype == kBF16)
        return launch_attention_general_t((const __nv_bfloat16*)y, stride, q_col, (__nv_bfloat16*)out, out_stride, out_col, out_scale,
                                          (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, positions, token_seq,
                                          block_table, table_stride, n_seqs, n_pages, n_tokens, heads, kv_heads, dim, v_dim,
                                          page_size, window, chunk, scale, status, stream);
    return launch_attention_general_t((const float*)y, stride, q_col, (float*)out, out_stride, out_col, out_scale, (const float*)k_cache,
                                      (const float*)v_cache, positions, token_seq, block_table, table_stride, n_seqs, n_pages,
                                      n_tokens, heads, kv_heads, dim, v_dim, page_size, window, chunk, scale, status, stream);
}

}  // namespace vtb
