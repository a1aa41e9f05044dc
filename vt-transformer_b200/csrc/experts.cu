// Mixture of experts: the routing step between the two packed products.
//
// The experts' gate and up matrices are one packed matrix and their down matrices are packed along the inner dimension,
// so a token's feed-forward is two products over all experts; what makes it a mixture is this kernel between them.  One
// block a token: a warp picks the `top` largest router logits (32-bit; the lower index among equals), forms the softmax
// over the picked logits, and the block multiplies the picked experts' columns of the activation by their weights and
// clears the others', so that the second product adds up exactly the chosen experts' results.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace vtb {

namespace {
constexpr int kMaxExperts = 1024;
constexpr int kRouteThreads = 128;
}

template <typename T>
__global__ void __launch_bounds__(kRouteThreads)
route_experts_kernel(const float* __restrict__ logits, int experts, int top, T* __restrict__ act, int act_stride, int inter) {
    __shared__ float z[kMaxExperts];          // the logits; a picked one is taken out
    __shared__ float w[kMaxExperts];          // the experts' weights, zero for those not picked
    __shared__ float picked_z[kMaxExperts];
    __shared__ int picked[kMaxExperts];
    pdl_launch();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        z[e] = logits[(size_t)t * experts + e];
        w[e] = 0.f;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int e = lane; e < experts; e += 32) {
                const float v = z[e];
                if (at == 0x7fffffff || v > best) { best = v; at = e; }      // a lane meets its experts in rising order
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (oa != 0x7fffffff && (at == 0x7fffffff || ov > best || (ov == best && oa < at))) { best = ov; at = oa; }
            }
            if (lane == 0) {
                picked[k] = at;
                picked_z[k] = best;
                z[at] = -INFINITY;
            }
            __syncwarp();
        }
        if (lane == 0) {
            const float mx = picked_z[0];                  // the first pick is the largest
            float sum = 0.f;
            for (int k = 0; k < top; ++k) sum += expf(picked_z[k] - mx);
            for (int k = 0; k < top; ++k) w[picked[k]] = expf(picked_z[k] - mx) / sum;
        }
    }
    __syncthreads();
    T* row = act + (size_t)t * act_stride;
    if (inter % 8 == 0 && act_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(act) & 15) == 0) {
        const int per = inter / 8;
        for (int c = threadIdx.x; c < experts * per; c += blockDim.x) {
            const float we = w[c / per];
            float v[8];
            if (we > 0.f) {
                Vec8<T>::load(row + c * 8, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= we;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 0.f;
            }
            Vec8<T>::store(row + c * 8, v);
        }
        return;
    }
    for (int c = threadIdx.x; c < experts * inter; c += blockDim.x) {
        const float we = w[c / inter];
        row[c] = from_float<T>(we > 0.f ? to_float(row[c]) * we : 0.f);
    }
}

cudaError_t launch_route_experts(int dtype, const float* logits, int n_tokens, int experts, int top, void* act, int act_stride,
                                 int inter, cudaStream_t stream) {
    if (n_tokens == 0) return cudaSuccess;
    if (experts < 1 || experts > kMaxExperts || top < 1 || top > experts) return cudaErrorInvalidValue;
    if (dtype == kBF16)
        return launch(route_experts_kernel<__nv_bfloat16>, n_tokens, kRouteThreads, 0, stream, logits, experts, top,
                      (__nv_bfloat16*)act, act_stride, inter);
    return launch(route_experts_kernel<float>, n_tokens, kRouteThreads, 0, stream, logits, experts, top, (float*)act, act_stride, inter);
}

}  // namespace vtb
