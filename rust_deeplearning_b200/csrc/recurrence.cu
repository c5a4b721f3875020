// Recurrences with a float state S [dim][vdim] per sequence and head whose decay depends on the token, token by token.
//
//   selective state space (RDL_REC_SSM), per head h with group g(h):
//       dt_t = softplus(raw_t[h] + dt_bias[h]);   S_t = exp(-exp(A_log[h]) dt_t) S_(t-1) + dt_t B_t x_t^T;
//       y_t  = S_t^T C_t + D[h] x_t                       B, C [dim] of the head's group, x [vdim]
//   delta rule with a decay per key channel (RDL_REC_DELTA), per head h with key head j(h):
//       S <- g_t (.) S  (row i times g_t[i]);   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//       q, k, g, beta come prepared in float (rdl_delta_prepare): q and k unit vectors (q times dim^-1/2),
//       g_t[i] = exp(-exp(A_log[h]) softplus(raw_t[h, i] + dt_bias[h, i])), beta_t = sigmoid(raw_t[h]).
//
// The layout is that of the fixed-decay scan: a block owns 32 columns of one head's state of one sequence, thread
// (column, slice) keeps RPT rows of its column in registers, the slices' parts of a column's sums are added in the
// order of the slices.  Nothing depends on how many tokens a step brings or on what else is in the batch.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int REC_COLS = 32;

__device__ __forceinline__ float softplus_exact(float z) { return z > 20.f ? z : log1pf(expf(z)); }

template <typename T, int RPT, int MODE>
__global__ void __launch_bounds__(256) recurrence_scan_kernel(RecurrenceArgs a) {
    extern __shared__ float sm[];
    const int dim = a.dim, vdim = a.vdim;
    float* q_s = sm;                          // [dim]  the vector the state is read out with (C, or q)
    float* k_s = q_s + dim;                   // [dim]  the vector the state is written with (dt B, or k)
    float* g_s = k_s + dim;                   // [dim]  the decay of each row (delta rule)
    float* part = g_s + dim;                  // [slices][REC_COLS]
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * REC_COLS;
    const int row0 = a.seq_start[seq], n = a.seq_start[seq + 1] - row0;
    if (n <= 0) return;
    if (a.tok_pos[row0] < 0) return;          // a padding sequence of a fixed-size batch
    const int tid = threadIdx.x, j = tid & 31, r = tid >> 5, n_thr = blockDim.x;
    const int col = c0 + j;
    const bool col_ok = col < vdim;
    const int i0 = r * RPT;
    const int slices = (dim + RPT - 1) / RPT;
    const int kh = h / (a.n_heads / a.n_key_heads);
    float* S = a.state + (((long long)a.slots[seq] * a.n_heads + h) * dim) * vdim;
    float s_reg[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) s_reg[i] = (col_ok && i0 + i < dim) ? S[(long long)(i0 + i) * vdim + col] : 0.f;
    const T* rows = (const T*)a.rows;
    const float neg_a = MODE == RDL_REC_SSM ? -expf(a.a_log[h]) : 0.f;
    const float d_skip = (MODE == RDL_REC_SSM && a.d_skip) ? a.d_skip[h] : 0.f;
    const float dt_bias = MODE == RDL_REC_SSM ? a.dt_bias[h] : 0.f;

    for (int t = 0; t < n; ++t) {
        const long long row = row0 + t;
        float decay = 1.f, beta = 0.f;
        if (MODE == RDL_REC_SSM) {
            const T* xr = rows + row * a.row_stride;
            const float dt = softplus_exact(to_float(((const T*)a.dt_rows)[row * a.dt_stride + h]) + dt_bias);
            decay = expf(neg_a * dt);
            for (int i = tid; i < dim; i += n_thr) {
                k_s[i] = dt * to_float(xr[a.k_col + kh * dim + i]);
                q_s[i] = to_float(xr[a.q_col + kh * dim + i]);
            }
        } else {
            const long long kq = row * a.n_key_heads * dim + (long long)kh * dim;
            const long long gr = row * a.n_heads * dim + (long long)h * dim;
            for (int i = tid; i < dim; i += n_thr) {
                q_s[i] = a.q_f[kq + i];
                k_s[i] = a.k_f[kq + i];
                g_s[i] = a.g_f[gr + i];
            }
            beta = a.beta_f[row * a.n_heads + h];
        }
        const float v = col_ok ? to_float(rows[row * a.row_stride + a.v_col + h * vdim + col]) : 0.f;
        __syncthreads();
        float acc = 0.f;
        if (MODE == RDL_REC_SSM) {
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                if (i0 + i < dim) {
                    s_reg[i] = fmaf(decay, s_reg[i], k_s[i0 + i] * v);
                    acc = fmaf(s_reg[i], q_s[i0 + i], acc);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                if (i0 + i < dim) {
                    s_reg[i] *= g_s[i0 + i];
                    acc = fmaf(s_reg[i], k_s[i0 + i], acc);
                }
            }
            part[r * REC_COLS + j] = acc;
            __syncthreads();
            float sk = 0.f;
            for (int s = 0; s < slices; ++s) sk += part[s * REC_COLS + j];
            const float u = beta * (v - sk);
            acc = 0.f;
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                if (i0 + i < dim) {
                    s_reg[i] = fmaf(k_s[i0 + i], u, s_reg[i]);
                    acc = fmaf(s_reg[i], q_s[i0 + i], acc);
                }
            }
            __syncthreads();                  // every thread has read the first sums
        }
        part[r * REC_COLS + j] = acc;
        __syncthreads();
        if (r == 0 && col_ok) {
            float o = 0.f;
            for (int s = 0; s < slices; ++s) o += part[s * REC_COLS + j];
            if (MODE == RDL_REC_SSM) o = fmaf(d_skip, v, o);
            a.out[row * a.n_heads * vdim + (long long)h * vdim + col] = o;
        }
        // no barrier here: the next token's vectors go to q_s, k_s and g_s, which nobody reads after the barrier above,
        // and `part` is written again only after the next token's first barrier, which the readers here reach last
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i)
        if (col_ok && i0 + i < dim) S[(long long)(i0 + i) * vdim + col] = s_reg[i];
}

// A block per token, a warp per head at a time: unit vectors of the key heads' q and k, decays and betas of the heads.
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(DeltaPrepareArgs a) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const long long t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int dim = a.dim;
    const T* xr = (const T*)a.rows + t * a.row_stride;
    for (int item = warp; item < 2 * a.n_key_heads; item += warps) {
        const bool is_q = item < a.n_key_heads;
        const int kh = is_q ? item : item - a.n_key_heads;
        const T* src = xr + (is_q ? a.q_col : a.k_col) + kh * dim;
        float ss = 0.f;
        for (int i = lane; i < dim; i += 32) { const float v = to_float(src[i]); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float inv = (is_q ? a.q_scale : 1.0f) / sqrtf(ss + a.unit_eps);
        float* dst = (is_q ? a.q_f : a.k_f) + t * a.n_key_heads * dim + (long long)kh * dim;
        for (int i = lane; i < dim; i += 32) dst[i] = to_float(src[i]) * inv;
    }
    const T* dr = (const T*)a.decay_rows + t * a.decay_stride;
    for (int h = warp; h < a.n_heads; h += warps) {
        const float neg_a = -expf(a.a_log[h]);
        for (int i = lane; i < dim; i += 32) {
            const float z = to_float(dr[h * dim + i]) + rdl_load(a.dt_bias, h * dim + i, a.bias_dtype);
            a.g_f[t * a.n_heads * dim + (long long)h * dim + i] = expf(neg_a * softplus_exact(z));
        }
        if (lane == 0) a.beta_f[t * a.n_heads + h] = 1.0f / (1.0f + expf(-to_float(((const T*)a.beta_rows)[t * a.beta_stride + h])));
    }
}

template <typename T, int MODE>
int launch_scan(const RecurrenceArgs* a, cudaStream_t st) {
    const int dim = a->dim;
    int rpt = 4;
    while (rpt < 64 && (dim + rpt - 1) / rpt > 8) rpt *= 2;
    const int slices = (dim + rpt - 1) / rpt;
    RDL_REQUIRE(slices <= 8, "recurrence_scan: dim %d exceeds 512", dim);
    const int threads = 32 * slices;
    const size_t smem = (size_t)(3 * dim + slices * REC_COLS) * sizeof(float);
    const dim3 grid(a->n_seqs, a->n_heads, (a->vdim + REC_COLS - 1) / REC_COLS);
    cudaError_t e;
    switch (rpt) {
        case 4: e = rdl_launch(recurrence_scan_kernel<T, 4, MODE>, grid, dim3(threads), smem, st, *a); break;
        case 8: e = rdl_launch(recurrence_scan_kernel<T, 8, MODE>, grid, dim3(threads), smem, st, *a); break;
        case 16: e = rdl_launch(recurrence_scan_kernel<T, 16, MODE>, grid, dim3(threads), smem, st, *a); break;
        case 32: e = rdl_launch(recurrence_scan_kernel<T, 32, MODE>, grid, dim3(threads), smem, st, *a); break;
        default: e = rdl_launch(recurrence_scan_kernel<T, 64, MODE>, grid, dim3(threads), smem, st, *a); break;
    }
    RDL_CHECK_EX(e, "recurrence_scan");
    return 0;
}

}  // namespace

extern "C" int rdl_recurrence_scan(const RecurrenceArgs* a, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(a->dtype), "recurrence_scan: bad dtype %d", a->dtype);
    RDL_REQUIRE(a->mode == RDL_REC_SSM || a->mode == RDL_REC_DELTA, "recurrence_scan: unknown mode %d", a->mode);
    RDL_REQUIRE(a->n_tokens >= 0 && a->n_seqs >= 0 && a->n_heads > 0 && a->n_key_heads > 0 && a->n_heads % a->n_key_heads == 0 && a->dim > 0 &&
                a->vdim > 0, "recurrence_scan: bad sizes");
    RDL_REQUIRE(a->rows && a->tok_pos && a->seq_start && a->slots && a->state && a->out, "recurrence_scan: missing rows, batch description, state or output");
    if (a->mode == RDL_REC_SSM)
        RDL_REQUIRE(a->dt_rows && a->dt_bias && a->a_log, "recurrence_scan: the state space form needs step sizes, their bias and A_log");
    else
        RDL_REQUIRE(a->q_f && a->k_f && a->g_f && a->beta_f, "recurrence_scan: the delta rule needs prepared q, k, decays and betas");
    RDL_REQUIRE(a->n_heads <= 65535 && (a->vdim + REC_COLS - 1) / REC_COLS <= 65535, "recurrence_scan: too many heads or columns for one grid");
    if (a->n_tokens == 0 || a->n_seqs == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->dtype == RDL_BF16)
        return a->mode == RDL_REC_SSM ? launch_scan<__nv_bfloat16, RDL_REC_SSM>(a, st) : launch_scan<__nv_bfloat16, RDL_REC_DELTA>(a, st);
    return a->mode == RDL_REC_SSM ? launch_scan<float, RDL_REC_SSM>(a, st) : launch_scan<float, RDL_REC_DELTA>(a, st);
}

extern "C" int rdl_delta_prepare(const DeltaPrepareArgs* a, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(a->dtype) && rdl_valid_dtype(a->bias_dtype), "delta_prepare: bad dtype");
    RDL_REQUIRE(a->n_tokens >= 0 && a->n_heads > 0 && a->n_key_heads > 0 && a->dim > 0, "delta_prepare: bad sizes");
    RDL_REQUIRE(a->rows && a->decay_rows && a->beta_rows && a->dt_bias && a->a_log && a->q_f && a->k_f && a->g_f && a->beta_f,
                "delta_prepare: missing rows, parameters or outputs");
    if (a->n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (a->dtype == RDL_BF16) RDL_CHECK_EX(rdl_launch(delta_prepare_kernel<__nv_bfloat16>, dim3(a->n_tokens), dim3(128), 0, st, *a), "delta_prepare");
    else RDL_CHECK_EX(rdl_launch(delta_prepare_kernel<float>, dim3(a->n_tokens), dim3(128), 0, st, *a), "delta_prepare");
    return 0;
}
