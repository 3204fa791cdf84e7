// tcnn::default_rng_t stand-in: PCG32 (O'Neill 2014; the generator tiny-cuda-nn ships as pcg32.h),
// written from the published algorithm: 64-bit LCG state, XSH-RR output, advance() by square-and-multiply,
// next_float() from the top 23 bits.  Host build of the test oracle only.
#pragma once
#include "common.h"
namespace tcnn {
struct pcg32 {
    static constexpr uint64_t kDefaultState = 0x853c49e6748fea9bULL, kDefaultStream = 0xda3e39cb94b95bdbULL,
                              kMult = 0x5851f42d4c957f2dULL;
    uint64_t state, inc;
    SRF_TCNN_HD pcg32() : state(kDefaultState), inc(kDefaultStream) {}
    SRF_TCNN_HD pcg32(uint64_t initstate, uint64_t initseq = 1u) { seed(initstate, initseq); }
    SRF_TCNN_HD void seed(uint64_t initstate, uint64_t initseq = 1) {
        state = 0u; inc = (initseq << 1u) | 1u;
        next_uint(); state += initstate; next_uint();
    }
    SRF_TCNN_HD uint32_t next_uint() {
        const uint64_t oldstate = state;
        state = oldstate * kMult + inc;
        const uint32_t xorshifted = (uint32_t)(((oldstate >> 18u) ^ oldstate) >> 27u);
        const uint32_t rot = (uint32_t)(oldstate >> 59u);
        return (xorshifted >> rot) | (xorshifted << ((~rot + 1u) & 31));
    }
    SRF_TCNN_HD float next_float() {
        union { uint32_t u; float f; } x;
        x.u = (next_uint() >> 9) | 0x3f800000u;
        return x.f - 1.0f;
    }
    SRF_TCNN_HD void advance(int64_t delta_ = (1ll << 32)) {
        uint64_t cur_mult = kMult, cur_plus = inc, acc_mult = 1u, acc_plus = 0u;
        uint64_t delta = (uint64_t)delta_;
        while (delta > 0) {
            if (delta & 1) { acc_mult *= cur_mult; acc_plus = acc_plus * cur_mult + cur_plus; }
            cur_plus = (cur_mult + 1) * cur_plus;
            cur_mult *= cur_mult;
            delta /= 2;
        }
        state = acc_mult * state + acc_plus;
    }
};
using default_rng_t = pcg32;
}  // namespace tcnn
