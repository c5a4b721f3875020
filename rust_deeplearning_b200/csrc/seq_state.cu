// Row kernels that look one or a few tokens back along a sequence and keep what they need of earlier steps per slot.
//
// norm_shift:  n_t = x_t / sqrt(mean(x_t^2) + eps) * w;   m_t = n_t + (n_(t-1) - n_t) * shift   (n_(-1) = 0)
//              the norm and the mix in float; the slot keeps n of the sequence's last token.
// short_conv:  y_t[c] = act(b[c] + sum_j w[c][j] x_(t-(K-1-j))[c])  (inputs before the sequence's start are zero)
//              the sum in float in the order of the taps; the slot keeps the last K - 1 inputs.
//
// Both are cut-invariant by construction: a value that comes from the slot was formed by the same operations in
// the same order as the value a longer step would have read from its own rows.  Only the block that owns a
// sequence's first row of the step touches the slot (it reads the old state, then writes the new one, element by
// element in the thread that read it), so a step's blocks need no order among themselves; with a convolution the
// first rows of a sequence, which all read the slot, are that block's too.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

__device__ __forceinline__ float silu_exact(float z) { return z / (1.0f + expf(-z)); }

// sum of squares of a float row, every thread gets it
__device__ __forceinline__ float row_square_sum(const float* __restrict__ x, int width, float* scratch) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    return block_sum(ss, scratch);
}

template <typename T>
__global__ void __launch_bounds__(256) norm_shift_kernel(const float* __restrict__ x, const void* __restrict__ w, int w_dtype, float eps,
                                                         const void* __restrict__ shift, int shift_dtype, float* __restrict__ state,
                                                         const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                                         const int* __restrict__ seq_start, const int* __restrict__ slots,
                                                         T* __restrict__ normed, T* __restrict__ mixed, int width) {
    __shared__ float scratch[33];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x;
    const float* xr = x + (long long)t * width;
    const float inv = 1.0f / sqrtf(row_square_sum(xr, width, scratch) / (float)width + eps);
    const int p = tok_pos[t];
    if (p < 0) {   // a padding row of a fixed-size batch: finite values, no slot
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const T v = from_float<T>(xr[i] * inv * rdl_load(w, i, w_dtype));
            normed[(long long)t * width + i] = v;
            mixed[(long long)t * width + i] = v;
        }
        return;
    }
    const int seq = tok_seq[t], row0 = seq_start[seq];
    const bool first = t == row0;
    float inv_prev = 0.f;
    const float* xp = xr - width;
    if (!first) inv_prev = 1.0f / sqrtf(row_square_sum(xp, width, scratch) / (float)width + eps);
    float* st = state + (long long)slots[seq] * width;
    const int last = seq_start[seq + 1] - 1;
    float inv_last = inv;
    const float* xl = x + (long long)last * width;
    if (first && last != t) inv_last = 1.0f / sqrtf(row_square_sum(xl, width, scratch) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float wi = rdl_load(w, i, w_dtype);
        const float n = xr[i] * inv * wi;
        float prev;
        if (!first) prev = xp[i] * inv_prev * wi;
        else prev = p == 0 ? 0.f : st[i];
        normed[(long long)t * width + i] = from_float<T>(n);
        mixed[(long long)t * width + i] = from_float<T>(n + (prev - n) * rdl_load(shift, i, shift_dtype));
        if (first) st[i] = xl[i] * inv_last * wi;
    }
}

constexpr int CONV_MAX_TAPS = 8;

// One row's outputs for the block's channels.  r: the row's index within its sequence's rows of this step.
template <typename T>
__device__ __forceinline__ void conv_row(const T* __restrict__ in, long long in_stride, int row0, int r, int past, int c, int channels,
                                         int taps, const float (&wt)[CONV_MAX_TAPS], float bias, int silu, const float (&old)[CONV_MAX_TAPS],
                                         T* __restrict__ out) {
    float acc = bias;
    for (int j = 0; j < taps; ++j) {
        const int src = r - (taps - 1 - j);
        float v;
        if (src >= 0) v = to_float(in[(long long)(row0 + src) * in_stride + c]);
        else v = past + src < 0 ? 0.f : old[taps - 1 + src];
        acc = fmaf(wt[j], v, acc);
    }
    out[(long long)(row0 + r) * channels + c] = from_float<T>(silu ? silu_exact(acc) : acc);
}

template <typename T>
__global__ void __launch_bounds__(128) short_conv_kernel(const T* __restrict__ in, long long in_stride, int channels, int taps,
                                                         const void* __restrict__ w, int w_dtype, const void* __restrict__ b, int silu,
                                                         float* __restrict__ state, const int* __restrict__ tok_seq,
                                                         const int* __restrict__ tok_pos, const int* __restrict__ seq_start,
                                                         const int* __restrict__ slots, T* __restrict__ out) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int p = tok_pos[t];
    if (p < 0) { out[(long long)t * channels + c] = from_float<T>(0.f); return; }
    const int seq = tok_seq[t], row0 = seq_start[seq], r = t - row0;
    if (r > 0 && r < taps - 1) return;          // the block of the sequence's first row forms these rows
    float wt[CONV_MAX_TAPS], old[CONV_MAX_TAPS];
    for (int j = 0; j < taps; ++j) wt[j] = rdl_load(w, (long long)c * taps + j, w_dtype);
    const float bias = b ? rdl_load(b, c, w_dtype) : 0.f;
    for (int j = 0; j < CONV_MAX_TAPS; ++j) old[j] = 0.f;
    if (r > 0) {                                 // every input lies in the step's own rows
        conv_row<T>(in, in_stride, row0, r, p - r, c, channels, taps, wt, bias, silu, old, out);
        return;
    }
    const int n = seq_start[seq + 1] - row0, keep = taps - 1;
    float* st = state + (long long)slots[seq] * keep * channels;
    if (p > 0)
        for (int j = 0; j < keep; ++j) old[j] = st[(long long)j * channels + c];
    for (int rr = 0; rr < min(n, max(keep, 1)); ++rr) conv_row<T>(in, in_stride, row0, rr, p, c, channels, taps, wt, bias, silu, old, out);
    for (int j = 0; j < keep; ++j) {
        const int src = n - keep + j;
        float v;
        if (src >= 0) v = to_float(in[(long long)(row0 + src) * in_stride + c]);
        else v = p + src < 0 ? 0.f : old[keep + src];
        st[(long long)j * channels + c] = v;
    }
}

template <typename T>
__global__ void gated_residual_kernel(float* __restrict__ res, const T* __restrict__ gates, long long gates_stride,
                                      const void* __restrict__ bias_a, const void* __restrict__ bias_b, int bias_dtype,
                                      const T* __restrict__ a, const T* __restrict__ b1, const T* __restrict__ b2, int width, long long total) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / width;
        const int i = (int)(idx - t * width);
        const float ga = to_float(gates[t * gates_stride + i]) + rdl_load(bias_a, i, bias_dtype);
        float sum = to_float(a[idx]) / (1.0f + expf(-ga));
        if (b1) {
            const float gb = to_float(gates[t * gates_stride + width + i]) + rdl_load(bias_b, i, bias_dtype);
            float f = to_float(b1[idx]);
            if (b2) f += to_float(b2[idx]);
            sum += f / (1.0f + expf(-gb));
        }
        res[idx] += sum;
    }
}

// the same sum for bfloat16 rows whose width is a multiple of 8: eight elements a thread, 16-byte accesses, one division
// by the width a thread instead of a 64-bit one an element; every element goes through the same operations as above
__global__ void __launch_bounds__(256) gated_residual_vec_kernel(float* __restrict__ res, const __nv_bfloat16* __restrict__ gates, long long gates_stride,
                                                                 const void* __restrict__ bias_a, const void* __restrict__ bias_b, int bias_dtype,
                                                                 const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b1,
                                                                 const __nv_bfloat16* __restrict__ b2, int width, int groups) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int per_row = width >> 3;
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < groups; v += gridDim.x * blockDim.x) {
        const int t = v / per_row, i = (v - t * per_row) << 3;
        const long long idx = (long long)t * width + i;
        const uint4 ga4 = *reinterpret_cast<const uint4*>(gates + t * gates_stride + i);
        const uint4 a4 = *reinterpret_cast<const uint4*>(a + idx);
        uint4 gb4 = make_uint4(0, 0, 0, 0), b14 = gb4, b24 = gb4;
        if (b1) {
            gb4 = *reinterpret_cast<const uint4*>(gates + t * gates_stride + width + i);
            b14 = *reinterpret_cast<const uint4*>(b1 + idx);
            if (b2) b24 = *reinterpret_cast<const uint4*>(b2 + idx);
        }
        float4 r0 = *reinterpret_cast<const float4*>(res + idx), r1 = *reinterpret_cast<const float4*>(res + idx + 4);
        const __nv_bfloat16* gav = reinterpret_cast<const __nv_bfloat16*>(&ga4);
        const __nv_bfloat16* gbv = reinterpret_cast<const __nv_bfloat16*>(&gb4);
        const __nv_bfloat16* av = reinterpret_cast<const __nv_bfloat16*>(&a4);
        const __nv_bfloat16* b1v = reinterpret_cast<const __nv_bfloat16*>(&b14);
        const __nv_bfloat16* b2v = reinterpret_cast<const __nv_bfloat16*>(&b24);
        float o[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float ga = __bfloat162float(gav[e]) + rdl_load(bias_a, i + e, bias_dtype);
            float sum = __bfloat162float(av[e]) / (1.0f + expf(-ga));
            if (b1) {
                const float gb = __bfloat162float(gbv[e]) + rdl_load(bias_b, i + e, bias_dtype);
                float f = __bfloat162float(b1v[e]);
                if (b2) f += __bfloat162float(b2v[e]);
                sum += f / (1.0f + expf(-gb));
            }
            o[e] += sum;
        }
        *reinterpret_cast<float4*>(res + idx) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4*>(res + idx + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
}

template <typename T>
__global__ void activation_kernel(T* __restrict__ x, long long total, int act) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const float v = to_float(x[idx]);
        float o;
        switch (act) {
            case RDL_UNARY_RELU2: { const float r = fmaxf(v, 0.f); o = r * r; break; }
            case RDL_UNARY_SILU: o = silu_exact(v); break;
            default: o = v;
        }
        x[idx] = from_float<T>(o);
    }
}

}  // namespace

extern "C" int rdl_norm_shift(const float* x, const void* w, int w_dtype, float eps, const void* shift, int shift_dtype, float* state,
                              const int* tok_seq, const int* tok_pos, const int* seq_start, const int* slots, void* normed, void* mixed,
                              int out_dtype, int n_rows, int width, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(out_dtype) && rdl_valid_dtype(w_dtype) && rdl_valid_dtype(shift_dtype), "norm_shift: bad dtype");
    RDL_REQUIRE(x && w && shift && state && tok_seq && tok_pos && seq_start && slots && normed && mixed && width > 0 && n_rows >= 0,
                "norm_shift: bad arguments");
    if (n_rows == 0) return 0;
    const dim3 grid(n_rows), block(width <= 512 ? 64 : (width <= 2048 ? 128 : 256));
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(norm_shift_kernel<__nv_bfloat16>, grid, block, 0, st, x, w, w_dtype, eps, shift, shift_dtype, state, tok_seq, tok_pos,
                                seq_start, slots, (__nv_bfloat16*)normed, (__nv_bfloat16*)mixed, width), "norm_shift");
    else
        RDL_CHECK_EX(rdl_launch(norm_shift_kernel<float>, grid, block, 0, st, x, w, w_dtype, eps, shift, shift_dtype, state, tok_seq, tok_pos,
                                seq_start, slots, (float*)normed, (float*)mixed, width), "norm_shift");
    return 0;
}

extern "C" int rdl_short_conv(const void* in, long long in_stride, int dtype, int channels, int taps, const void* w, int w_dtype,
                              const void* bias, int silu, float* state, const int* tok_seq, const int* tok_pos, const int* seq_start,
                              const int* slots, void* out, int n_rows, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype) && rdl_valid_dtype(w_dtype), "short_conv: bad dtype");
    RDL_REQUIRE(in && w && tok_seq && tok_pos && seq_start && slots && out && channels > 0 && in_stride >= channels && n_rows >= 0,
                "short_conv: bad arguments");
    RDL_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "short_conv: %d taps, the kernel takes 1 to %d", taps, CONV_MAX_TAPS);
    RDL_REQUIRE(state || taps == 1, "short_conv: more than one tap needs the slots' state");
    if (n_rows == 0) return 0;
    RDL_REQUIRE((channels + 127) / 128 <= 65535, "short_conv: too many channels for one grid");
    const dim3 grid(n_rows, (channels + 127) / 128), block(128);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(short_conv_kernel<__nv_bfloat16>, grid, block, 0, st, (const __nv_bfloat16*)in, in_stride, channels, taps, w, w_dtype,
                                bias, silu, state, tok_seq, tok_pos, seq_start, slots, (__nv_bfloat16*)out), "short_conv");
    else
        RDL_CHECK_EX(rdl_launch(short_conv_kernel<float>, grid, block, 0, st, (const float*)in, in_stride, channels, taps, w, w_dtype, bias, silu,
                                state, tok_seq, tok_pos, seq_start, slots, (float*)out), "short_conv");
    return 0;
}

extern "C" int rdl_gated_residual_add(float* res, const void* gates, long long gates_stride, const void* bias_a, const void* bias_b,
                                      int bias_dtype, const void* a, const void* b1, const void* b2, int dtype, int n_rows, int width,
                                      void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype) && rdl_valid_dtype(bias_dtype), "gated_residual_add: bad dtype");
    RDL_REQUIRE(res && gates && bias_a && a && width > 0 && n_rows >= 0 && (!b1 || bias_b) && (b1 || !b2), "gated_residual_add: bad arguments");
    RDL_REQUIRE(gates_stride >= (b1 ? 2LL : 1LL) * width, "gated_residual_add: the gates' rows are narrower than the branches");
    if (n_rows == 0) return 0;
    const long long total = (long long)n_rows * width;
    const dim3 grid((unsigned)min((total + 255) / 256, 65535LL * 16)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
    const bool aligned = (((uintptr_t)res | (uintptr_t)gates | (uintptr_t)a | (uintptr_t)b1 | (uintptr_t)b2) & 15) == 0;
    if (dtype == RDL_BF16 && width % 8 == 0 && gates_stride % 8 == 0 && aligned && total / 8 < (1LL << 31)) {
        const int groups = (int)(total / 8);
        RDL_CHECK_EX(rdl_launch(gated_residual_vec_kernel, dim3((unsigned)min((groups + 255) / 256, 148 * 16)), block, 0, st, res, (const __nv_bfloat16*)gates,
                                gates_stride, bias_a, bias_b, bias_dtype, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b1, (const __nv_bfloat16*)b2, width, groups),
                     "gated_residual_add");
    } else if (dtype == RDL_BF16)
        RDL_CHECK_EX(rdl_launch(gated_residual_kernel<__nv_bfloat16>, grid, block, 0, st, res, (const __nv_bfloat16*)gates, gates_stride, bias_a, bias_b,
                                bias_dtype, (const __nv_bfloat16*)a, (const __nv_bfloat16*)b1, (const __nv_bfloat16*)b2, width, total),
                     "gated_residual_add");
    else
        RDL_CHECK_EX(rdl_launch(gated_residual_kernel<float>, grid, block, 0, st, res, (const float*)gates, gates_stride, bias_a, bias_b, bias_dtype,
                                (const float*)a, (const float*)b1, (const float*)b2, width, total), "gated_residual_add");
    return 0;
}

extern "C" int rdl_activation_inplace(void* x, int dtype, long long total, int act, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(dtype) && x && total >= 0, "activation_inplace: bad arguments");
    RDL_REQUIRE(act == RDL_UNARY_RELU2 || act == RDL_UNARY_SILU, "activation_inplace: unknown activation %d", act);
    if (total == 0) return 0;
    const dim3 grid((unsigned)min((total + 255) / 256, 65535LL * 16)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == RDL_BF16) RDL_CHECK_EX(rdl_launch(activation_kernel<__nv_bfloat16>, grid, block, 0, st, (__nv_bfloat16*)x, total, act), "activation_inplace");
    else RDL_CHECK_EX(rdl_launch(activation_kernel<float>, grid, block, 0, st, (float*)x, total, act), "activation_inplace");
    return 0;
}
