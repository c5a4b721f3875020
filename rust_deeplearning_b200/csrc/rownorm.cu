// Row kernels of designs that norm after the sum, gate a mixer's output element by element, or average two
// normed branches.  Statistics and products are float; a row is one block's, and the order of its sums depends
// on the row's width alone (never on how many rows a step has).
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

__device__ __forceinline__ float gate_value(float g, int act) {
    const float s = 1.0f / (1.0f + expf(-g));
    return act == RDL_GATE_SILU ? g * s : s;
}

// For results that are rounded to bfloat16 anyway: the hardware's exponential and reciprocal (a few units in the last
// place of a float, far below a bfloat16's half unit).
__device__ __forceinline__ float gate_value_fast(float g, int act) {
    const float s = __fdividef(1.0f, 1.0f + __expf(-g));
    return act == RDL_GATE_SILU ? g * s : s;
}

// Four consecutive values at a time, and a row (or group) held in registers between its two passes: every load of a
// thread is asked for before the first is used, so a row costs one trip to memory however wide it is.  Used when
// the width is a multiple of 4 and a thread's share fits RN_MAX_IT groups of four; the plain loops further down serve the rest.
#define RN_MAX_IT 8
__device__ __forceinline__ void rn_load4(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
__device__ __forceinline__ void rn_load4(const __nv_bfloat16* p, float (&f)[4]) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void rn_load4(const void* p, long long i, int dtype, float (&f)[4]) {
    if (dtype == RDL_BF16) rn_load4((const __nv_bfloat16*)p + i, f); else rn_load4((const float*)p + i, f);
}
__device__ __forceinline__ void rn_store4(float* p, const float (&f)[4]) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
__device__ __forceinline__ void rn_store4(__nv_bfloat16* p, const float (&f)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&a); raw.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}
// threads of a block whose row is `width` wide: a multiple of 32 that depends on the width alone
static inline int vec_threads(int width) {
    const int groups = width / 4;
    int t = (groups + RN_MAX_IT - 1) / RN_MAX_IT;      // the fewest that keep a thread's share within RN_MAX_IT
    if (t < (groups + 1) / 2) t = (groups + 1) / 2;    // but two groups a thread at most while a block holds them
    t = (t + 31) / 32 * 32;
    return t > 256 ? 256 : (t < 32 ? 32 : t);
}
static inline bool vec_ok(int width, int threads) { return width % 4 == 0 && (width / 4 + threads - 1) / threads <= RN_MAX_IT; }
static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
// groups of four a thread takes, rounded up to 1, 2, 4 or 8 (the kernels' unrolled depth)
static inline int vec_depth(int width, int threads) {
    const int need = (width / 4 + threads - 1) / threads;
    return need <= 1 ? 1 : (need <= 2 ? 2 : (need <= 4 ? 4 : 8));
}
#define RN_BY_DEPTH(depth, LAUNCH) \
    switch (depth) { case 1: LAUNCH(1); break; case 2: LAUNCH(2); break; case 4: LAUNCH(4); break; default: LAUNCH(8); break; }

template <typename TB, typename TY, int NIT>
__global__ void __launch_bounds__(256) postnorm_vec_kernel(float* __restrict__ res, const TB* __restrict__ branch, float alpha,
                                                           const void* __restrict__ w, int w_dtype, float eps, float off,
                                                           TY* __restrict__ y, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    float* r = res + (long long)blockIdx.x * width;
    const TB* b = branch + (long long)blockIdx.x * width;
    float h[NIT][4], bv[NIT][4];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) { rn_load4(r + e, h[it]); rn_load4(b + e, bv[it]); }
    }
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) {
#pragma unroll
            for (int k = 0; k < 4; ++k) { h[it][k] = fmaf(alpha, h[it][k], bv[it][k]); ss = fmaf(h[it][k], h[it][k], ss); }
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) {
            float wv[4], v[4];
            rn_load4(w, e, w_dtype, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = h[it][k] * inv * (wv[k] + off);
            rn_store4(r + e, v);
            if (y) rn_store4(y + (long long)blockIdx.x * width + e, v);
        }
    }
}

template <typename T, int NIT>
__global__ void __launch_bounds__(256) norm_pair_vec_kernel(float* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b,
                                                            const void* __restrict__ wa, const void* __restrict__ wb, int w_dtype,
                                                            float eps, float c, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const T* ra = a + (long long)blockIdx.x * width;
    const T* rb = b + (long long)blockIdx.x * width;
    float x[NIT][4], z[NIT][4];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) { rn_load4(ra + e, x[it]); rn_load4(rb + e, z[it]); }
    }
    float sa = 0.f, sb = 0.f;
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) {
#pragma unroll
            for (int k = 0; k < 4; ++k) { sa = fmaf(x[it][k], x[it][k], sa); sb = fmaf(z[it][k], z[it][k], sb); }
        }
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = 1.0f / sqrtf(sa / (float)width + eps), ib = 1.0f / sqrtf(sb / (float)width + eps);
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) {
            float va[4], vb[4], v[4];
            rn_load4(wa, e, w_dtype, va);
            rn_load4(wb, e, w_dtype, vb);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = c * (x[it][k] * ia * va[k] + z[it][k] * ib * vb[k]);
            rn_store4(out + (long long)blockIdx.x * width + e, v);
        }
    }
}

// a warp per group (groups of up to 1,024 values), or a block per group (WARP false)
template <typename TO, bool WARP, int NIT>
__global__ void __launch_bounds__(256) group_norm_gate_vec_kernel(TO* __restrict__ out, const float* __restrict__ x, long long n_items, int groups,
                                                                  int group, const void* __restrict__ w, int w_dtype, float eps,
                                                                  const void* __restrict__ g, long long g_stride, int g_dtype, int act,
                                                                  int gate_first) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const long long item = WARP ? (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) : blockIdx.x;
    if (WARP && item >= n_items) return;
    const int lane = WARP ? (threadIdx.x & 31) : threadIdx.x, stride = WARP ? 32 : blockDim.x;
    const long long t = item / groups;
    const int gi = (int)(item - t * groups), col0 = gi * group;
    const long long base = item * group;
    float v[NIT][4], gv[NIT][4];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (lane + it * stride) * 4;
        if (e < group) {
            rn_load4(x + base + e, v[it]);
            if (g) rn_load4(g, t * g_stride + col0 + e, g_dtype, gv[it]);
            if (g && gate_first) {
#pragma unroll
                for (int k = 0; k < 4; ++k) v[it][k] *= gate_value(gv[it][k], act);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (lane + it * stride) * 4;
        if (e < group) {
#pragma unroll
            for (int k = 0; k < 4; ++k) ss = fmaf(v[it][k], v[it][k], ss);
        }
    }
    ss = WARP ? warp_sum(ss) : block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)group + eps);
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (lane + it * stride) * 4;
        if (e < group) {
            float o[4], wv[4];
            if (w) rn_load4(w, col0 + e, w_dtype, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                o[k] = v[it][k] * inv;
                if (w) o[k] *= wv[k];
                if (g && !gate_first) o[k] *= sizeof(TO) == 2 ? gate_value_fast(gv[it][k], act) : gate_value(gv[it][k], act);
            }
            rn_store4(out + base + e, o);
        }
    }
}

static inline int row_threads(int width) { return width <= 256 ? 64 : (width <= 2048 ? 128 : 256); }

// res <- norm(alpha * res + branch); y (optional) the same rows in another type
template <typename TB, typename TY>
__global__ void postnorm_kernel(float* __restrict__ res, const TB* __restrict__ branch, float alpha, const void* __restrict__ w,
                                int w_dtype, float eps, float off, TY* __restrict__ y, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    float* r = res + (long long)blockIdx.x * width;
    const TB* b = branch + (long long)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float h = fmaf(alpha, r[i], to_float(b[i]));
        r[i] = h;                     // this thread reads it back below
        ss = fmaf(h, h, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = r[i] * inv * (rdl_load(w, i, w_dtype) + off);
        r[i] = v;
        if (y) y[(long long)blockIdx.x * width + i] = from_float<TY>(v);
    }
}

extern "C" int rdl_postnorm(float* res, const void* branch, int branch_dtype, float alpha, const void* w, int w_dtype, float eps,
                            float off, void* y, int y_dtype, int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(branch_dtype) && rdl_valid_dtype(w_dtype) && rdl_valid_dtype(y_dtype), "postnorm: bad dtype");
    RDL_REQUIRE(res && branch && w && n_rows >= 0 && width > 0, "postnorm: missing rows or weight");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const int vt = vec_threads(width);
    if (vec_ok(width, vt) && aligned16(res) && aligned16(branch) && aligned16(w) && aligned16(y)) {
        const dim3 grid(n_rows), block(vt);
#define POSTNORM_LAUNCH(N)                                                                                                          \
    do {                                                                                                                            \
        if (branch_dtype == RDL_BF16) {                                                                                             \
            if (y_dtype == RDL_BF16)                                                                                                \
                e = rdl_launch(postnorm_vec_kernel<__nv_bfloat16, __nv_bfloat16, N>, grid, block, 0, st, res,                       \
                               (const __nv_bfloat16*)branch, alpha, w, w_dtype, eps, off, (__nv_bfloat16*)y, width);                \
            else                                                                                                                    \
                e = rdl_launch(postnorm_vec_kernel<__nv_bfloat16, float, N>, grid, block, 0, st, res, (const __nv_bfloat16*)branch, \
                               alpha, w, w_dtype, eps, off, (float*)y, width);                                                      \
        } else {                                                                                                                    \
            if (y_dtype == RDL_BF16)                                                                                                \
                e = rdl_launch(postnorm_vec_kernel<float, __nv_bfloat16, N>, grid, block, 0, st, res, (const float*)branch, alpha,  \
                               w, w_dtype, eps, off, (__nv_bfloat16*)y, width);                                                     \
            else                                                                                                                    \
                e = rdl_launch(postnorm_vec_kernel<float, float, N>, grid, block, 0, st, res, (const float*)branch, alpha, w,       \
                               w_dtype, eps, off, (float*)y, width);                                                                \
        }                                                                                                                           \
    } while (0)
        RN_BY_DEPTH(vec_depth(width, vt), POSTNORM_LAUNCH)
#undef POSTNORM_LAUNCH
        RDL_CHECK_EX(e, "postnorm");
        return 0;
    }
    const dim3 grid(n_rows), block(row_threads(width));
    if (branch_dtype == RDL_BF16) {
        if (y_dtype == RDL_BF16)
            e = rdl_launch(postnorm_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, st, res, (const __nv_bfloat16*)branch, alpha, w,
                           w_dtype, eps, off, (__nv_bfloat16*)y, width);
        else
            e = rdl_launch(postnorm_kernel<__nv_bfloat16, float>, grid, block, 0, st, res, (const __nv_bfloat16*)branch, alpha, w, w_dtype,
                           eps, off, (float*)y, width);
    } else {
        if (y_dtype == RDL_BF16)
            e = rdl_launch(postnorm_kernel<float, __nv_bfloat16>, grid, block, 0, st, res, (const float*)branch, alpha, w, w_dtype, eps,
                           off, (__nv_bfloat16*)y, width);
        else
            e = rdl_launch(postnorm_kernel<float, float>, grid, block, 0, st, res, (const float*)branch, alpha, w, w_dtype, eps, off,
                           (float*)y, width);
    }
    RDL_CHECK_EX(e, "postnorm");
    return 0;
}

// out = c (norm(a; wa) + norm(b; wb))
template <typename T>
__global__ void norm_pair_kernel(float* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, const void* __restrict__ wa,
                                 const void* __restrict__ wb, int w_dtype, float eps, float c, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const T* ra = a + (long long)blockIdx.x * width;
    const T* rb = b + (long long)blockIdx.x * width;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = to_float(ra[i]), z = to_float(rb[i]);
        sa = fmaf(x, x, sa);
        sb = fmaf(z, z, sb);
    }
    sa = block_sum(sa, scratch);
    sb = block_sum(sb, scratch);
    const float ia = 1.0f / sqrtf(sa / (float)width + eps), ib = 1.0f / sqrtf(sb / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float x = to_float(ra[i]) * ia * rdl_load(wa, i, w_dtype);
        const float z = to_float(rb[i]) * ib * rdl_load(wb, i, w_dtype);
        out[(long long)blockIdx.x * width + i] = c * (x + z);
    }
}

extern "C" int rdl_norm_pair(float* out, const void* a, const void* b, int dtype, const void* wa, const void* wb, int w_dtype,
                             float eps, float c, int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype) && rdl_valid_dtype(w_dtype), "norm_pair: bad dtype");
    RDL_REQUIRE(out && a && b && wa && wb && n_rows >= 0 && width > 0, "norm_pair: missing rows or weights");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const int vt = vec_threads(width);
    if (vec_ok(width, vt) && aligned16(out) && aligned16(a) && aligned16(b) && aligned16(wa) && aligned16(wb)) {
#define NORM_PAIR_LAUNCH(N)                                                                                                  \
    do {                                                                                                                     \
        if (dtype == RDL_BF16)                                                                                               \
            e = rdl_launch(norm_pair_vec_kernel<__nv_bfloat16, N>, dim3(n_rows), dim3(vt), 0, st, out, (const __nv_bfloat16*)a, \
                           (const __nv_bfloat16*)b, wa, wb, w_dtype, eps, c, width);                                         \
        else                                                                                                                 \
            e = rdl_launch(norm_pair_vec_kernel<float, N>, dim3(n_rows), dim3(vt), 0, st, out, (const float*)a, (const float*)b, \
                           wa, wb, w_dtype, eps, c, width);                                                                  \
    } while (0)
        RN_BY_DEPTH(vec_depth(width, vt), NORM_PAIR_LAUNCH)
#undef NORM_PAIR_LAUNCH
        RDL_CHECK_EX(e, "norm_pair");
        return 0;
    }
    if (dtype == RDL_BF16)
        e = rdl_launch(norm_pair_kernel<__nv_bfloat16>, dim3(n_rows), dim3(row_threads(width)), 0, st, out, (const __nv_bfloat16*)a,
                       (const __nv_bfloat16*)b, wa, wb, w_dtype, eps, c, width);
    else
        e = rdl_launch(norm_pair_kernel<float>, dim3(n_rows), dim3(row_threads(width)), 0, st, out, (const float*)a, (const float*)b, wa,
                       wb, w_dtype, eps, c, width);
    RDL_CHECK_EX(e, "norm_pair");
    return 0;
}


template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ out, long long out_stride, const T* __restrict__ x, long long x_stride,
                                const T* __restrict__ g, long long g_stride, int act, int n_rows, int width) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const long long total = (long long)n_rows * width;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / width;
        const int i = (int)(idx - t * width);
        out[t * out_stride + i] = from_float<T>(to_float(x[t * x_stride + i]) * gate_value(to_float(g[t * g_stride + i]), act));
    }
}

// the same, eight bfloat16 values (16 bytes) a thread; width and the three strides are multiples of 8
__global__ void gate_mul_vec_kernel(__nv_bfloat16* __restrict__ out, long long out_stride, const __nv_bfloat16* __restrict__ x, long long x_stride,
                                    const __nv_bfloat16* __restrict__ g, long long g_stride, int act, int n_rows, int width) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int per_row = width >> 3;
    const long long total = (long long)n_rows * per_row;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / per_row;
        const int i = (int)(idx - t * per_row) << 3;
        const uint4 xr = *reinterpret_cast<const uint4*>(x + t * x_stride + i), gr = *reinterpret_cast<const uint4*>(g + t * g_stride + i);
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xr);
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gr);
        uint4 o;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 xv = __bfloat1622float2(xp[k]), gv = __bfloat1622float2(gp[k]);
            op[k] = __floats2bfloat162_rn(xv.x * gate_value_fast(gv.x, act), xv.y * gate_value_fast(gv.y, act));
        }
        *reinterpret_cast<uint4*>(out + t * out_stride + i) = o;
    }
}

extern "C" int rdl_gate_mul(void* out, long long out_stride, const void* x, long long x_stride, const void* g, long long g_stride,
                            int dtype, int gate_act, int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype), "gate_mul: bad dtype %d", dtype);
    RDL_REQUIRE(gate_act == RDL_GATE_SIGMOID || gate_act == RDL_GATE_SILU, "gate_mul: unknown gate %d", gate_act);
    RDL_REQUIRE(out && x && g && n_rows >= 0 && width > 0 && out_stride >= width && x_stride >= width && g_stride >= width,
                "gate_mul: missing rows or strides below the width");
    if (n_rows == 0) return 0;
    const long long total = (long long)n_rows * width;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 65535 * 8 ? (total + 255) / 256 : 65535 * 8);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (dtype == RDL_BF16 && width % 8 == 0 && out_stride % 8 == 0 && x_stride % 8 == 0 && g_stride % 8 == 0 && aligned16(out) &&
        aligned16(x) && aligned16(g)) {
        const long long groups = total / 8;
        const unsigned vblocks = (unsigned)((groups + 255) / 256 < 65535 * 8 ? (groups + 255) / 256 : 65535 * 8);
        e = rdl_launch(gate_mul_vec_kernel, dim3(vblocks), dim3(256), 0, st, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)x, x_stride,
                       (const __nv_bfloat16*)g, g_stride, gate_act, n_rows, width);
        RDL_CHECK_EX(e, "gate_mul");
        return 0;
    }
    if (dtype == RDL_BF16)
        e = rdl_launch(gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st, (__nv_bfloat16*)out, out_stride,
                       (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)g, g_stride, gate_act, n_rows, width);
    else
        e = rdl_launch(gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, st, (float*)out, out_stride, (const float*)x, x_stride,
                       (const float*)g, g_stride, gate_act, n_rows, width);
    RDL_CHECK_EX(e, "gate_mul");
    return 0;
}

// float rows normed group by group, times an optional weight and an optional gate
template <typename TO>
__global__ void group_norm_gate_kernel(TO* __restrict__ out, const float* __restrict__ x, int groups, int group, const void* __restrict__ w,
                                       int w_dtype, float eps, const void* __restrict__ g, long long g_stride, int g_dtype, int act,
                                       int gate_first) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x, gi = blockIdx.y;
    const long long base = ((long long)t * groups + gi) * group;
    const int col0 = gi * group;
    float ss = 0.f;
    const bool first = g && gate_first;
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        float v = x[base + i];
        if (first) v *= gate_value(rdl_load(g, (long long)t * g_stride + col0 + i, g_dtype), act);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)group + eps);
    for (int i = threadIdx.x; i < group; i += blockDim.x) {
        float v = x[base + i];
        if (first) v *= gate_value(rdl_load(g, (long long)t * g_stride + col0 + i, g_dtype), act);
        v *= inv;
        if (w) v *= rdl_load(w, col0 + i, w_dtype);
        if (g && !first) v *= gate_value(rdl_load(g, (long long)t * g_stride + col0 + i, g_dtype), act);
        out[base + i] = from_float<TO>(v);
    }
}

extern "C" int rdl_group_norm_gate(void* out, int out_dtype, const float* x, int n_rows, int groups, int group, const void* w,
                                   int w_dtype, float eps, const void* g, long long g_stride, int g_dtype, int gate_act, int gate_first,
                                   void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(out_dtype) && rdl_valid_dtype(w_dtype) && rdl_valid_dtype(g_dtype), "group_norm_gate: bad dtype");
    RDL_REQUIRE(out && x && n_rows >= 0 && groups > 0 && groups <= 65535 && group > 0, "group_norm_gate: bad sizes");
    RDL_REQUIRE(gate_act == RDL_GATE_SIGMOID || gate_act == RDL_GATE_SILU, "group_norm_gate: unknown gate %d", gate_act);
    RDL_REQUIRE(!g || g_stride >= (long long)groups * group, "group_norm_gate: the gate's rows are narrower than the groups");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const long long n_items = (long long)n_rows * groups;
    const bool all16 = aligned16(out) && aligned16(x) && aligned16(w) && aligned16(g) && (!g || g_stride % 8 == 0);
    if (all16 && group % 8 == 0 && n_items < (1LL << 31)) {
        const bool warp = group <= 4 * 32 * RN_MAX_IT;
        const int vt = vec_threads(group);
        if (warp || vec_ok(group, vt)) {
            const dim3 grid(warp ? (unsigned)((n_items + 7) / 8) : (unsigned)n_items), block(warp ? 256 : vt);
#define GROUP_NORM_LAUNCH(N)                                                                                                             \
    do {                                                                                                                                 \
        if (out_dtype == RDL_BF16) {                                                                                                     \
            if (warp) e = rdl_launch(group_norm_gate_vec_kernel<__nv_bfloat16, true, N>, grid, block, 0, st, (__nv_bfloat16*)out, x,     \
                                     n_items, groups, group, w, w_dtype, eps, g, g_stride, g_dtype, gate_act, gate_first);               \
            else e = rdl_launch(group_norm_gate_vec_kernel<__nv_bfloat16, false, N>, grid, block, 0, st, (__nv_bfloat16*)out, x,         \
                                n_items, groups, group, w, w_dtype, eps, g, g_stride, g_dtype, gate_act, gate_first);                    \
        } else {                                                                                                                         \
            if (warp) e = rdl_launch(group_norm_gate_vec_kernel<float, true, N>, grid, block, 0, st, (float*)out, x, n_items, groups,    \
                                     group, w, w_dtype, eps, g, g_stride, g_dtype, gate_act, gate_first);                                \
            else e = rdl_launch(group_norm_gate_vec_kernel<float, false, N>, grid, block, 0, st, (float*)out, x, n_items, groups, group, \
                                w, w_dtype, eps, g, g_stride, g_dtype, gate_act, gate_first);                                            \
        }                                                                                                                                \
    } while (0)
            RN_BY_DEPTH(vec_depth(group, warp ? 32 : vt), GROUP_NORM_LAUNCH)
#undef GROUP_NORM_LAUNCH
            RDL_CHECK_EX(e, "group_norm_gate");
            return 0;
        }
    }
    const dim3 grid(n_rows, groups), block(group <= 64 ? 32 : row_threads(group));
    if (out_dtype == RDL_BF16)
        e = rdl_launch(group_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, st, (__nv_bfloat16*)out, x, groups, group, w, w_dtype, eps, g,
                       g_stride, g_dtype, gate_act, gate_first);
    else
        e = rdl_launch(group_norm_gate_kernel<float>, grid, block, 0, st, (float*)out, x, groups, group, w, w_dtype, eps, g, g_stride,
                       g_dtype, gate_act, gate_first);
    RDL_CHECK_EX(e, "group_norm_gate");
    return 0;
}

// ---- the sum of a block whose sublayers read one norm, with the norm the next part asks for ----
// res <- res + scale * (a + b + c) (b, c optional), then y <- norm(res) if y is given.  The branches are added up in
// float in the order a, b, c; a row's sum of squares is formed in an order that depends on its width alone.
template <typename TB, typename TY, int NIT>
__global__ void __launch_bounds__(256) add_branches_norm_vec_kernel(float* __restrict__ res, const TB* __restrict__ a, const TB* __restrict__ b,
                                                                    const TB* __restrict__ c, float scale, const void* __restrict__ w,
                                                                    int w_dtype, float eps, float off, TY* __restrict__ y, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const long long base = (long long)blockIdx.x * width;
    float h[NIT][4], av[NIT][4], bv[NIT][4], cv[NIT][4];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) {
            rn_load4(res + base + e, h[it]);
            rn_load4(a + base + e, av[it]);
            if (b) rn_load4(b + base + e, bv[it]);
            if (c) rn_load4(c + base + e, cv[it]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float s = av[it][k];
                if (b) s += bv[it][k];
                if (c) s += cv[it][k];
                h[it][k] = fmaf(scale, s, h[it][k]);
                ss = fmaf(h[it][k], h[it][k], ss);
            }
            rn_store4(res + base + e, h[it]);
        }
    }
    if (!y) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int e = (threadIdx.x + it * blockDim.x) * 4;
        if (e < width) {
            float wv[4], v[4];
            rn_load4(w, e, w_dtype, wv);
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = h[it][k] * inv * (wv[k] + off);
            rn_store4(y + base + e, v);
        }
    }
}

template <typename TB, typename TY>
__global__ void add_branches_norm_kernel(float* __restrict__ res, const TB* __restrict__ a, const TB* __restrict__ b, const TB* __restrict__ c,
                                         float scale, const void* __restrict__ w, int w_dtype, float eps, float off, TY* __restrict__ y,
                                         int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const long long base = (long long)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float s = to_float(a[base + i]);
        if (b) s += to_float(b[base + i]);
        if (c) s += to_float(c[base + i]);
        const float h = fmaf(scale, s, res[base + i]);
        res[base + i] = h;            // this thread reads it back below
        ss = fmaf(h, h, ss);
    }
    if (!y) return;
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        y[base + i] = from_float<TY>(res[base + i] * inv * (rdl_load(w, i, w_dtype) + off));
}

extern "C" int rdl_add_branches_norm(float* res, const void* a, const void* b, const void* c, int branch_dtype, float scale, const void* w,
                                     int w_dtype, float eps, float off, void* y, int y_dtype, int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(branch_dtype) && rdl_valid_dtype(w_dtype) && rdl_valid_dtype(y_dtype), "add_branches_norm: bad dtype");
    RDL_REQUIRE(res && a && n_rows >= 0 && width > 0 && (!y || w), "add_branches_norm: missing rows, branch or weight");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    const int vt = vec_threads(width);
    const dim3 grid(n_rows);
    const bool vec = vec_ok(width, vt) && aligned16(res) && aligned16(a) && aligned16(b) && aligned16(c) && aligned16(w) && aligned16(y);
    const int depth = vec_depth(width, vt);
#define ABN_VEC(TB, TY, N) \
    e = rdl_launch(add_branches_norm_vec_kernel<TB, TY, N>, grid, dim3(vt), 0, st, res, (const TB*)a, (const TB*)b, (const TB*)c, scale, w, w_dtype, eps, off, (TY*)y, width)
#define ABN_LAUNCH(N)                                                                       \
    do {                                                                                    \
        if (branch_dtype == RDL_BF16) {                                                     \
            if (y_dtype == RDL_BF16) ABN_VEC(__nv_bfloat16, __nv_bfloat16, N);              \
            else ABN_VEC(__nv_bfloat16, float, N);                                          \
        } else {                                                                            \
            if (y_dtype == RDL_BF16) ABN_VEC(float, __nv_bfloat16, N);                      \
            else ABN_VEC(float, float, N);                                                  \
        }                                                                                   \
    } while (0)
#define ABN_PLAIN(TB, TY) \
    e = rdl_launch(add_branches_norm_kernel<TB, TY>, grid, dim3(row_threads(width)), 0, st, res, (const TB*)a, (const TB*)b, (const TB*)c, scale, w, w_dtype, eps, off, (TY*)y, width)
    if (vec) {
        RN_BY_DEPTH(depth, ABN_LAUNCH)
    } else if (branch_dtype == RDL_BF16) {
        if (y_dtype == RDL_BF16) ABN_PLAIN(__nv_bfloat16, __nv_bfloat16); else ABN_PLAIN(__nv_bfloat16, float);
    } else {
        if (y_dtype == RDL_BF16) ABN_PLAIN(float, __nv_bfloat16); else ABN_PLAIN(float, float);
    }
#undef ABN_VEC
#undef ABN_LAUNCH
#undef ABN_PLAIN
    RDL_CHECK_EX(e, "add_branches_norm");
    return 0;
}
