// srf_cuda_on_host.h -- the few CUDA device built-ins the reference's kernels use, defined for host
// compilation by the test oracle's build (oracle/build_ref.py).  TEST INFRASTRUCTURE ONLY.
//
// Host builds: a kernel becomes an ordinary function; the harness sets threadIdx/blockIdx/blockDim before each call
// and runs the "threads" in index order.  Under nvcc (the GPU build of the same kernels, baseline/) only the surface
// stand-in below is defined: everything else is the real thing there.  __expf/__logf are the C library's expf/logf
// here (the GPU's are approximations with documented error bounds; no host code can reproduce their bits).
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <cassert>
#include <string>
#include <vector>
#include <algorithm>
#include <stdexcept>
#include <iostream>

#include <cuda_runtime.h>      // vector types, dim3, qualifier macros for host compilers
#include <cuda_fp16.h>         // __half with host conversions

#if !defined(__CUDACC__)
// ---- host compilation: the built-ins as ordinary functions ---------------------------------------------------------
struct SrfThreadIndex { unsigned int x = 0, y = 0, z = 0; };
extern thread_local SrfThreadIndex threadIdx, blockIdx;
extern thread_local SrfThreadIndex blockDim, gridDim;

inline float __expf(float x) { return expf(x); }
inline float __logf(float x) { return logf(x); }
inline float __powf(float x, float y) { return powf(x, y); }
inline unsigned int __float_as_uint(float f) { unsigned int u; memcpy(&u, &f, 4); return u; }
inline float __uint_as_float(unsigned int u) { float f; memcpy(&f, &u, 4); return f; }

// "threads" run one after another, so plain read-modify-write is atomic enough
inline unsigned int atomicAdd(unsigned int* p, unsigned int v) { const unsigned int o = *p; *p = o + v; return o; }
inline unsigned int atomicMax(unsigned int* p, unsigned int v) { const unsigned int o = *p; if (v > o) *p = v; return o; }
inline float atomicAdd(float* p, float v) { const float o = *p; *p = o + v; return o; }

// integer min/max with CUDA's mixed signed/unsigned overloads
inline int min(int a, int b) { return a < b ? a : b; }
inline int max(int a, int b) { return a < b ? b : a; }
inline unsigned int min(unsigned int a, unsigned int b) { return a < b ? a : b; }
inline unsigned int max(unsigned int a, unsigned int b) { return a < b ? b : a; }
inline unsigned int min(unsigned int a, int b) { return min(a, (unsigned int)b); }
inline unsigned int min(int a, unsigned int b) { return min((unsigned int)a, b); }
inline unsigned int max(unsigned int a, int b) { return max(a, (unsigned int)b); }
inline unsigned int max(int a, unsigned int b) { return max((unsigned int)a, b); }
inline float min(float a, float b) { return fminf(a, b); }
inline float max(float a, float b) { return fmaxf(a, b); }

#endif   // !__CUDACC__

// tonemap_kernel writes its pixel through a surface; here the "surface" is a float4 image in host memory
struct SrfHostSurface { float4* pixels; int width; };
typedef SrfHostSurface* srf_surface_t;
#define cudaSurfaceObject_t srf_surface_t
#if defined(__CUDACC__)
__host__ __device__
#endif
inline void surf2Dwrite(float4 v, srf_surface_t s, int x_bytes, int y) { s->pixels[(size_t)y * s->width + x_bytes / (int)sizeof(float4)] = v; }
