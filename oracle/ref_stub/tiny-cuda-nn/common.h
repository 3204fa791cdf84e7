// Stand-ins for the few tiny-cuda-nn helpers the reference's kernels call (host build of the test oracle;
// see ../srf_cuda_on_host.h).  tiny-cuda-nn itself is not available; these follow its published behaviour:
// fp16 network precision, clamp, logistic 1/(1+exp(-x)), logit -log(1/x-1), bit-interleaving Morton codes,
// a fixed-size aligned vector.
#pragma once
#include "../srf_cuda_on_host.h"

#if defined(__CUDACC__)
#define SRF_TCNN_HD __host__ __device__
#else
#define SRF_TCNN_HD
#endif

namespace tcnn {

using network_precision_t = __half;

template <typename T> SRF_TCNN_HD inline T clamp(T val, T lower, T upper) { return val < lower ? lower : (upper < val ? upper : val); }
template <typename T> SRF_TCNN_HD inline void host_device_swap(T& a, T& b) { T c(a); a = b; b = c; }
template <typename T> SRF_TCNN_HD inline T div_round_up(T val, T divisor) { return (val + divisor - 1) / divisor; }
template <typename T> SRF_TCNN_HD inline T next_multiple(T val, T divisor) { return div_round_up(val, divisor) * divisor; }

SRF_TCNN_HD inline float logistic(const float x) { return 1.0f / (1.0f + expf(-x)); }
SRF_TCNN_HD inline float logit(const float x) { return -logf(1.0f / x - 1.0f); }

SRF_TCNN_HD inline uint32_t expand_bits(uint32_t v) {
    v = (v * 0x00010001u) & 0xFF0000FFu;
    v = (v * 0x00000101u) & 0x0F00F00Fu;
    v = (v * 0x00000011u) & 0xC30C30C3u;
    v = (v * 0x00000005u) & 0x49249249u;
    return v;
}
SRF_TCNN_HD inline uint32_t morton3D(uint32_t x, uint32_t y, uint32_t z) { return expand_bits(x) | (expand_bits(y) << 1) | (expand_bits(z) << 2); }
SRF_TCNN_HD inline uint32_t morton3D_invert(uint32_t x) {
    x = x & 0x49249249u;
    x = (x | (x >> 2)) & 0xc30c30c3u;
    x = (x | (x >> 4)) & 0x0f00f00fu;
    x = (x | (x >> 8)) & 0xff0000ffu;
    x = (x | (x >> 16)) & 0x0000ffffu;
    return x;
}

template <typename T, uint32_t N>
struct alignas(sizeof(T) * N) vector_t {
    T data[N];
    SRF_TCNN_HD T& operator[](uint32_t i) { return data[i]; }
    SRF_TCNN_HD const T& operator[](uint32_t i) const { return data[i]; }
};

}  // namespace tcnn
