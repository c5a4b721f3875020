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
// The state space form and delta rules with heads of more than 256 rows take the layout of the fixed-decay scan: a block
// owns 32 columns of one head's state of one sequence, thread (column, slice) keeps RPT rows of its column in registers,
// the slices' parts of a column's sums are added in the order of the slices.  The delta rule with smaller heads, where
// every token has two sums one after the other, takes four warps per eight columns (delta_rule_kernel below).
// Nothing depends on how many tokens a step brings or on what else is in the batch.
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

// ---- the delta rule: a block of four warps per eight columns, a warp per two ----
constexpr int DR_COLS = 8;          // columns of a block
constexpr int DR_STAGES = 8;        // tokens whose prepared vectors are in shared memory or on their way there
constexpr int DR_THREADS = 128;

__device__ __forceinline__ void dr_copy16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_copy4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dr_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void dr_wait_oldest() { asm volatile("cp.async.wait_group %0;" ::"n"(DR_STAGES - 2) : "memory"); }
__device__ __forceinline__ void dr_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// A stage of the ring, in floats: q, k and g, each as sixteen slices of RPS rows (a slice starts 16 bytes after the one
// before it would end where that keeps eight slices' 16-byte reads in different banks); then the block's eight values of
// v as they lie in the rows (16 or 32 bytes) and beta.
template <int RPS> struct DrStage {
    static constexpr int SLICE = RPS == 4 ? 4 : RPS + 4, VEC = 16 * SLICE, V = 3 * VEC, BETA = V + 8, FLOATS = V + 12;
    __device__ static __forceinline__ int at(int i) { return (i / RPS) * SLICE + (i % RPS); }
};

// what a thread copies for every token: warps 0, 1, 2 the vectors q, k, g (lane l the values 4 l .. 4 l + 3 and, for heads
// of more than 128 rows, 128 further on), warp 3 the values of v and beta
template <typename T, int RPS>
struct DrSource {
    const float* vec; long long vec_step; int off; bool two;      // warps 0..2, rows in steps of 16 bytes
    const char* v; long long v_step; bool has_v;                  // warp 3, lanes 0 (and 1)
    const float* beta; long long beta_step;                       // warp 3, lane 31
};

template <typename T, int RPS>
__device__ __forceinline__ void dr_ask(const RecurrenceArgs& a, const DrSource<T, RPS>& src, int t, float* stage, int warp, int lane,
                                       long long row, int h, int kh, bool wide) {
    using L = DrStage<RPS>;
    if (warp < 3) {
        if (wide) {
            if (4 * lane < a.dim) dr_copy16(stage + warp * L::VEC + src.off, src.vec + t * src.vec_step);
            if (RPS > 8 && src.two) dr_copy16(stage + warp * L::VEC + L::at(4 * lane + 128), src.vec + t * src.vec_step + 128);
        } else {
            const float* from = warp == 0 ? a.q_f + (row * a.n_key_heads + kh) * a.dim : warp == 1 ? a.k_f + (row * a.n_key_heads + kh) * a.dim
                                                                                                  : a.g_f + (row * a.n_heads + h) * a.dim;
            for (int i = lane; i < a.dim; i += 32) dr_copy4(stage + warp * L::VEC + L::at(i), from + i);
        }
    } else {
        if (src.has_v) dr_copy16(reinterpret_cast<char*>(stage + L::V) + 16 * lane, src.v + t * src.v_step);
        if (lane == 31) dr_copy4(stage + L::BETA, src.beta + t * src.beta_step);
    }
}

// Lane (column c = lane / 16, slice r = lane % 16) of warp w keeps rows r RPS .. r RPS + RPS - 1 of column 2 w + c of the
// block in registers; a column's sums are the lane's partial sums and four exchanges among the column's sixteen lanes, the
// same tree for every token.  The prepared vectors of the next tokens are on their way into shared memory (asynchronous
// copies, a group a token, shared by the four warps) while a token is worked on: the chain from one token's state to the
// next holds no load from global memory, and a block has one barrier a token.
template <typename T, int RPS>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(RecurrenceArgs a) {
    using L = DrStage<RPS>;
    extern __shared__ __align__(16) float dr_ring[];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int dim = a.dim, vdim = a.vdim;
    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DR_COLS;
    const int row0 = a.seq_start[seq], n = a.seq_start[seq + 1] - row0;
    if (n <= 0) return;
    if (a.tok_pos[row0] < 0) return;          // a padding sequence of a fixed-size batch
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kh = h / (a.n_heads / a.n_key_heads);
    const int c = lane >> 4, r = lane & 15, bc = 2 * warp + c, col = c0 + bc;
    const bool col_ok = col < vdim;
    const unsigned full = 0xffffffffu;
    const T* rows = (const T*)a.rows;
    const bool wide = (dim & 3) == 0 && (((uintptr_t)a.q_f | (uintptr_t)a.k_f | (uintptr_t)a.g_f) & 15) == 0;
    const bool v_wide = c0 + DR_COLS <= vdim && (a.row_stride * sizeof(T)) % 16 == 0 &&
                        ((uintptr_t)(rows + (long long)row0 * a.row_stride + a.v_col + h * vdim + c0) & 15) == 0;
    DrSource<T, RPS> src;
    src.vec = warp == 0 ? a.q_f + ((long long)row0 * a.n_key_heads + kh) * dim : warp == 1 ? a.k_f + ((long long)row0 * a.n_key_heads + kh) * dim
                                                                                         : a.g_f + ((long long)row0 * a.n_heads + h) * dim;
    src.vec += 4 * lane;
    src.vec_step = (long long)(warp < 2 ? a.n_key_heads : a.n_heads) * dim;
    src.off = L::at(4 * lane < 16 * RPS ? 4 * lane : 0);
    src.two = 4 * lane + 128 < dim;
    src.v = reinterpret_cast<const char*>(rows + (long long)row0 * a.row_stride + a.v_col + h * vdim + c0) + 16 * lane;
    src.v_step = a.row_stride * (long long)sizeof(T);
    src.has_v = v_wide && lane < (int)(DR_COLS * sizeof(T) / 16);
    src.beta = a.beta_f + (long long)row0 * a.n_heads + h;
    src.beta_step = a.n_heads;
    // The block's eight columns of the state come through shared memory: two lanes fetch a row's 32 bytes side by side, so
    // that a step of single tokens, which is nothing but this fetch and its store, moves whole sectors.
    float* tile = dr_ring + DR_STAGES * L::FLOATS;          // [16 RPS rows][9]
    float* Sb = a.state + (((long long)a.slots[seq] * a.n_heads + h) * dim) * vdim + c0;
    const bool s_wide = (vdim & 3) == 0 && c0 + DR_COLS <= vdim && ((uintptr_t)a.state & 15) == 0;
    for (int idx = tid; idx < 32 * RPS; idx += DR_THREADS) {
        const int row = idx >> 1, c4 = 4 * (idx & 1);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < dim) {
            const float* from = Sb + (long long)row * vdim + c4;
            if (s_wide) v = *reinterpret_cast<const float4*>(from);
            else {
                if (c0 + c4 < vdim) v.x = from[0];
                if (c0 + c4 + 1 < vdim) v.y = from[1];
                if (c0 + c4 + 2 < vdim) v.z = from[2];
                if (c0 + c4 + 3 < vdim) v.w = from[3];
            }
        }
        float* to = tile + row * 9 + c4;
        to[0] = v.x; to[1] = v.y; to[2] = v.z; to[3] = v.w;
    }
    // rows beyond the head's last: q = k = 0 and g = 1 in every stage, never written again
    if (dim < 16 * RPS) {
        for (int i = tid; i < DR_STAGES * L::FLOATS; i += DR_THREADS) {
            const int w = i % L::FLOATS;
            dr_ring[i] = (w >= 2 * L::VEC && w < 3 * L::VEC) ? 1.f : 0.f;
        }
    }
    __syncthreads();
#pragma unroll
    for (int d = 0; d < DR_STAGES - 1; ++d) {
        if (d < n) dr_ask<T, RPS>(a, src, d, dr_ring + d * L::FLOATS, warp, lane, row0 + d, h, kh, wide);
        dr_commit();
    }
    float s[RPS];
#pragma unroll
    for (int i = 0; i < RPS; ++i) s[i] = tile[(r * RPS + i) * 9 + bc];
    float* out = a.out + (long long)row0 * a.n_heads * vdim + (long long)h * vdim + col;
    const int out_step = a.n_heads * vdim;

    for (int t = 0; t < n; ++t) {
        const float* stage = dr_ring + (t % DR_STAGES) * L::FLOATS;
        dr_wait_oldest();
        __syncthreads();            // token t's vectors are there for every warp, and every warp is done with token t - 1's
        const int ahead = t + DR_STAGES - 1;
        if (ahead < n) dr_ask<T, RPS>(a, src, ahead, dr_ring + (ahead % DR_STAGES) * L::FLOATS, warp, lane, row0 + ahead, h, kh, wide);
        dr_commit();
        const float* qs = stage + r * L::SLICE;
        const float* ks = qs + L::VEC;
        const float* gs = ks + L::VEC;
        float kr[RPS], qr[RPS];
        float p0 = 0.f, p1 = 0.f;
#pragma unroll
        for (int i = 0; i < RPS; i += 4) {
            const float4 g4 = *reinterpret_cast<const float4*>(gs + i), k4 = *reinterpret_cast<const float4*>(ks + i);
            const float4 q4 = *reinterpret_cast<const float4*>(qs + i);
            kr[i] = k4.x; kr[i + 1] = k4.y; kr[i + 2] = k4.z; kr[i + 3] = k4.w;
            qr[i] = q4.x; qr[i + 1] = q4.y; qr[i + 2] = q4.z; qr[i + 3] = q4.w;
            s[i] *= g4.x; s[i + 1] *= g4.y; s[i + 2] *= g4.z; s[i + 3] *= g4.w;
            p0 = fmaf(s[i], k4.x, p0); p1 = fmaf(s[i + 1], k4.y, p1); p0 = fmaf(s[i + 2], k4.z, p0); p1 = fmaf(s[i + 3], k4.w, p1);
        }
        float v = 0.f;
        if (col_ok) v = v_wide ? to_float(reinterpret_cast<const T*>(stage + L::V)[bc]) : to_float(rows[(long long)(row0 + t) * a.row_stride + a.v_col + h * vdim + col]);
        const float beta = stage[L::BETA];
        float sk = p0 + p1;
        sk += __shfl_xor_sync(full, sk, 1);
        sk += __shfl_xor_sync(full, sk, 2);
        sk += __shfl_xor_sync(full, sk, 4);
        sk += __shfl_xor_sync(full, sk, 8);
        const float u = beta * (v - sk);
        float o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int i = 0; i < RPS; i += 2) {
            s[i] = fmaf(kr[i], u, s[i]);
            s[i + 1] = fmaf(kr[i + 1], u, s[i + 1]);
            o0 = fmaf(s[i], qr[i], o0);
            o1 = fmaf(s[i + 1], qr[i + 1], o1);
        }
        float y = o0 + o1;
        y += __shfl_xor_sync(full, y, 1);
        y += __shfl_xor_sync(full, y, 2);
        y += __shfl_xor_sync(full, y, 4);
        y += __shfl_xor_sync(full, y, 8);
        if (r == 0 && col_ok) out[(long long)t * out_step] = y;
    }
    dr_wait_all();
#pragma unroll
    for (int i = 0; i < RPS; ++i) tile[(r * RPS + i) * 9 + bc] = s[i];
    __syncthreads();
    for (int idx = tid; idx < 32 * RPS; idx += DR_THREADS) {
        const int row = idx >> 1, c4 = 4 * (idx & 1);
        if (row >= dim) continue;
        const float* from = tile + row * 9 + c4;
        float* to = Sb + (long long)row * vdim + c4;
        if (s_wide) *reinterpret_cast<float4*>(to) = make_float4(from[0], from[1], from[2], from[3]);
        else {
            if (c0 + c4 < vdim) to[0] = from[0];
            if (c0 + c4 + 1 < vdim) to[1] = from[1];
            if (c0 + c4 + 2 < vdim) to[2] = from[2];
            if (c0 + c4 + 3 < vdim) to[3] = from[3];
        }
    }
}

template <typename T, int RPS>
cudaError_t launch_delta_rule_rows(const RecurrenceArgs* a, cudaStream_t st) {
    const dim3 grid(a->n_seqs, a->n_heads, (a->vdim + DR_COLS - 1) / DR_COLS);
    return rdl_launch(delta_rule_kernel<T, RPS>, grid, dim3(DR_THREADS), (size_t)(DR_STAGES * DrStage<RPS>::FLOATS + 16 * RPS * 9) * sizeof(float), st, *a);
}

template <typename T>
int launch_delta_rule(const RecurrenceArgs* a, cudaStream_t st) {
    cudaError_t e;
    if (a->dim <= 64) e = launch_delta_rule_rows<T, 4>(a, st);
    else if (a->dim <= 128) e = launch_delta_rule_rows<T, 8>(a, st);
    else e = launch_delta_rule_rows<T, 16>(a, st);
    RDL_CHECK_EX(e, "recurrence_scan (delta rule)");
    return 0;
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
    if (MODE == RDL_REC_DELTA && dim <= 256) return launch_delta_rule<T>(a, st);
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
