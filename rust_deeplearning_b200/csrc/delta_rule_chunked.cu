// The delta rule with a decay per key channel, eight tokens at a time, in float throughout (the token-by-token form is
// recurrence.cu's).
//
// Per head, with S the state before a group of tokens 1..C (C = 8), g_t the decays, and P(j, t) = g_(j+1) (.) ... (.) g_t
// the decay of what token j wrote (j = 0: of S itself) until token t reads it:
//     S_t = g_t (.) S_(t-1) + k_t u_t^T,     u_t = beta_t (v_t - (g_t (.) S_(t-1))^T k_t),     o_t = S_t^T q_t
// unrolls into
//     u_t = beta_t (v_t - S^T kd_t - sum_(j<t) A_tj u_j)         kd_t = P(0, t) (.) k_t,   A_tj = sum_i k_t[i] k_j[i] P(j, t)[i]
//     o_t = S^T qd_t + sum_(j<=t) B_tj u_j                       qd_t = P(0, t) (.) q_t,   B_tj = sum_i q_t[i] k_j[i] P(j, t)[i]
//     S'  = P(0, C) (.) S + sum_j w_j u_j^T                      w_j  = P(j, C) (.) k_j
// Every P is a product of decays (never a quotient), so nothing overflows however small a decay is.  kd, qd, w, P(0, C), A
// and B depend on no state: a first launch makes them for all groups of the step at once (a record per group and head, laid
// out as the second launch reads it), together with beta and v in float.  The second launch walks each sequence's groups:
// a block of eight warps per 16 columns of a head's state, lane (column, slice) with RPS rows of its column in registers.
// For a group a lane forms its parts of the 16 sums S^T kd_t and S^T qd_t in one pass, the sixteen lanes of a column add
// them in one round of exchanges, u = T r and o = S^T qd + (B T) r follow as one row of products a lane (the triangular
// system's inverse T = (I + diag(beta) A)^-1 diag(beta) and B T depend on no state and come with the record), and the
// state takes all eight writes in one pass: two dependent passes and one round of exchanges per eight tokens instead of
// per token.  The records of the next groups are on their way into shared memory (asynchronous copies) meanwhile.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

constexpr int DC_C = 8;             // tokens of a group
constexpr int DC_COLS = 16;         // columns of a block of the second launch
constexpr int DC_THREADS = 256;
constexpr int DC_STAGES = 4;
constexpr int DC_SCALARS = 2 * DC_C * DC_C + DC_C;      // A, B, beta

// A record in floats: 3 C + 1 vectors (kd_t, qd_t, w_t for every t, then P(0, C)), each as sixteen slices of RPS rows (a
// slice starts 16 bytes after the one before it would end where that keeps eight slices' 16-byte reads in different banks);
// then T [C][C], B T [C][C], beta [C]; then v [C][columns rounded up to 16].
template <int RPS> struct DcRecord {
    static constexpr int SLICE = RPS == 4 ? 4 : RPS + 4, VEC = 16 * SLICE, SC = (3 * DC_C + 1) * VEC, V = SC + DC_SCALARS;
    static constexpr int STAGE = V + DC_C * DC_COLS;          // what a block keeps of a record
    __host__ __device__ static int at(int i) { return (i / RPS) * SLICE + (i % RPS); }
    __host__ __device__ static long long floats(int vdim) { return V + (long long)DC_C * ((vdim + DC_COLS - 1) / DC_COLS * DC_COLS); }
};

static inline int dc_max_groups(int n_tokens, int n_seqs) {
    const int by_tokens = n_tokens / DC_C + n_seqs;
    return by_tokens < n_tokens ? by_tokens : n_tokens;
}

// group number `idx` of the step -> its sequence and its first token there; false beyond the step's last group
__device__ __forceinline__ bool dc_find_group(const RecurrenceArgs& a, int idx, int& seq, int& t0) {
    for (int s = 0; s < a.n_seqs; ++s) {
        const int n = a.seq_start[s + 1] - a.seq_start[s];
        const int ng = (n > 0 && a.tok_pos[a.seq_start[s]] >= 0) ? (n + DC_C - 1) / DC_C : 0;
        if (idx < ng) { seq = s; t0 = idx * DC_C; return true; }
        idx -= ng;
    }
    return false;
}

// ---- first launch: a block per (group, head), a thread per key channel ----
template <typename T, int RPS>
__global__ void __launch_bounds__(128) dc_record_kernel(RecurrenceArgs a, float* __restrict__ records) {
    using R = DcRecord<RPS>;
    __shared__ float part[4][2 * DC_C * DC_C];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    int seq, t0;
    if (!dc_find_group(a, blockIdx.x, seq, t0)) return;
    const int h = blockIdx.y, dim = a.dim, vdim = a.vdim;
    const int kh = h / (a.n_heads / a.n_key_heads);
    const int row0 = a.seq_start[seq] + t0, L = min(DC_C, a.seq_start[seq + 1] - row0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float* rec = records + ((long long)blockIdx.x * a.n_heads + h) * R::floats(vdim);
    const bool live = tid < dim;
    float g[DC_C], k[DC_C], q[DC_C];
#pragma unroll
    for (int t = 0; t < DC_C; ++t) {
        const bool ok = live && t < L;
        const long long row = row0 + t;
        g[t] = ok ? a.g_f[(row * a.n_heads + h) * dim + tid] : 1.f;
        k[t] = ok ? a.k_f[(row * a.n_key_heads + kh) * dim + tid] : 0.f;
        q[t] = ok ? a.q_f[(row * a.n_key_heads + kh) * dim + tid] : 0.f;
    }
    // this channel's terms of A and B: for every writer j the running product of the decays after it
    float ab[2 * DC_C * DC_C];
#pragma unroll
    for (int i = 0; i < 2 * DC_C * DC_C; ++i) ab[i] = 0.f;
    float w[DC_C];
#pragma unroll
    for (int j = 0; j < DC_C; ++j) {
        ab[DC_C * DC_C + j * DC_C + j] = q[j] * k[j];
        float p = 1.f;
#pragma unroll
        for (int t = j + 1; t < DC_C; ++t) {
            p *= g[t];
            ab[t * DC_C + j] = k[t] * k[j] * p;
            ab[DC_C * DC_C + t * DC_C + j] = q[t] * k[j] * p;
        }
        w[j] = k[j] * p;
    }
    float p = 1.f;
    const int off = R::at(tid);
#pragma unroll
    for (int t = 0; t < DC_C; ++t) {
        p *= g[t];
        if (tid < 16 * RPS) {
            rec[t * R::VEC + off] = k[t] * p;
            rec[(DC_C + t) * R::VEC + off] = q[t] * p;
            rec[(2 * DC_C + t) * R::VEC + off] = w[t];
        }
    }
    if (tid < 16 * RPS) rec[3 * DC_C * R::VEC + off] = live ? p : 0.f;
    // sums over the channels: the lanes of a warp, then the four warps in their order
#pragma unroll
    for (int i = 0; i < 2 * DC_C * DC_C; ++i) {
        const int t = (i % (DC_C * DC_C)) / DC_C, j = i % DC_C;
        if (j > t || (j == t && i < DC_C * DC_C)) continue;      // never read
        const float s = warp_sum(ab[i]);
        if (lane == 0) part[warp][i] = s;
    }
    __syncthreads();
    __shared__ float fin[2 * DC_C * DC_C], tm[DC_C * DC_C], bet[DC_C];
    for (int i = tid; i < 2 * DC_C * DC_C; i += 128) {
        const int t = (i % (DC_C * DC_C)) / DC_C, j = i % DC_C;
        const bool used = j < t || (j == t && i >= DC_C * DC_C);
        fin[i] = used ? ((part[0][i] + part[1][i]) + (part[2][i] + part[3][i])) : 0.f;
    }
    if (tid < DC_C) bet[tid] = tid < L ? a.beta_f[(long long)(row0 + tid) * a.n_heads + h] : 0.f;
    __syncthreads();
    // u = T r with r_t = v_t - S^T kd_t and T = (I + diag(beta) A)^-1 diag(beta): thread j forms column j by substitution
    if (tid < DC_C) {
        const int j = tid;
        float x[DC_C];
#pragma unroll
        for (int t = 0; t < DC_C; ++t) x[t] = t == j ? 1.f : 0.f;
#pragma unroll
        for (int t = 1; t < DC_C; ++t) {
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < t; ++i) acc = fmaf(fin[t * DC_C + i], x[i], acc);
            if (t > j) x[t] = -bet[t] * acc;
        }
#pragma unroll
        for (int t = 0; t < DC_C; ++t) tm[t * DC_C + j] = x[t] * bet[j];
    }
    __syncthreads();
    // o = S^T qd + (B T) r
    if (tid < DC_C * DC_C) {
        const int t = tid / DC_C, j = tid % DC_C;
        float acc = 0.f;
        for (int i = j; i <= t; ++i) acc = fmaf(fin[DC_C * DC_C + t * DC_C + i], tm[i * DC_C + j], acc);
        rec[R::SC + tid] = tm[tid];
        rec[R::SC + DC_C * DC_C + tid] = acc;
    }
    if (tid < DC_C) rec[R::SC + 2 * DC_C * DC_C + tid] = bet[tid];
    const int vp = (vdim + DC_COLS - 1) / DC_COLS * DC_COLS;
    const T* rows = (const T*)a.rows;
    for (int i = tid; i < DC_C * vp; i += 128) {
        const int t = i / vp, c = i - t * vp;
        rec[R::V + i] = (t < L && c < vdim) ? to_float(rows[(long long)(row0 + t) * a.row_stride + a.v_col + h * vdim + c]) : 0.f;
    }
}

// ---- second launch ----
__device__ __forceinline__ void dc_copy16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void dc_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void dc_wait_oldest() { asm volatile("cp.async.wait_group %0;" ::"n"(DC_STAGES - 2) : "memory"); }
__device__ __forceinline__ void dc_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// a record's vectors and scalars, and this block's 16 columns of its v, into a stage
template <int RPS>
__device__ __forceinline__ void dc_ask(const float* rec, int vp, int c0, float* stage, int tid) {
    using R = DcRecord<RPS>;
    for (int i = 4 * tid; i < R::V; i += 4 * DC_THREADS) dc_copy16(stage + i, rec + i);
    if (tid < DC_C * DC_COLS / 4) {
        const int t = tid / (DC_COLS / 4), c = 4 * (tid % (DC_COLS / 4));
        dc_copy16(stage + R::V + t * DC_COLS + c, rec + R::V + (long long)t * vp + c0 + c);
    }
}

// Sixteen sums over the sixteen lanes of a column at once: halves are exchanged while the values a lane keeps halve (8, 4,
// 2, 1 lanes apart); lane r of the sixteen ends with the whole sum number r.
__device__ __forceinline__ float dc_sum16(const float (&x)[16], int r) {
    const unsigned full = 0xffffffffu;
    float y8[8], y4[4], y2[2];
    const bool b3 = r & 8, b2 = r & 4, b1 = r & 2, b0 = r & 1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float mine = b3 ? x[i + 8] : x[i], send = b3 ? x[i] : x[i + 8];
        y8[i] = mine + __shfl_xor_sync(full, send, 8);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float mine = b2 ? y8[i + 4] : y8[i], send = b2 ? y8[i] : y8[i + 4];
        y4[i] = mine + __shfl_xor_sync(full, send, 4);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float mine = b1 ? y4[i + 2] : y4[i], send = b1 ? y4[i] : y4[i + 2];
        y2[i] = mine + __shfl_xor_sync(full, send, 2);
    }
    const float mine = b0 ? y2[1] : y2[0], send = b0 ? y2[0] : y2[1];
    return mine + __shfl_xor_sync(full, send, 1);
}

template <int RPS>
__global__ void __launch_bounds__(DC_THREADS) dc_scan_kernel(RecurrenceArgs a, const float* __restrict__ records) {
    using R = DcRecord<RPS>;
    extern __shared__ __align__(16) float dc_ring[];
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int dim = a.dim, vdim = a.vdim;
    const int seq = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * DC_COLS;
    const int row0 = a.seq_start[seq], n = a.seq_start[seq + 1] - row0;
    if (n <= 0) return;
    if (a.tok_pos[row0] < 0) return;          // a padding sequence of a fixed-size batch
    int first = 0;                            // the step's groups before this sequence's
    for (int s = 0; s < seq; ++s) {
        const int m = a.seq_start[s + 1] - a.seq_start[s];
        if (m > 0 && a.tok_pos[a.seq_start[s]] >= 0) first += (m + DC_C - 1) / DC_C;
    }
    const int groups = (n + DC_C - 1) / DC_C;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c = lane >> 4, r = lane & 15, bc = 2 * warp + c, col = c0 + bc;
    const bool col_ok = col < vdim;
    const unsigned full = 0xffffffffu;
    const int vp = (vdim + DC_COLS - 1) / DC_COLS * DC_COLS;
    const long long rec_floats = R::floats(vdim);
    const float* rec0 = records + ((long long)first * a.n_heads + h) * rec_floats;
    const long long rec_step = (long long)a.n_heads * rec_floats;
#pragma unroll
    for (int d = 0; d < DC_STAGES - 1; ++d) {
        if (d < groups) dc_ask<RPS>(rec0 + d * rec_step, vp, c0, dc_ring + d * R::STAGE, tid);
        dc_commit();
    }
    float* S = a.state + (((long long)a.slots[seq] * a.n_heads + h) * dim) * vdim + col;
    float s[RPS];
#pragma unroll
    for (int i = 0; i < RPS; ++i) s[i] = (col_ok && r * RPS + i < dim) ? S[(long long)(r * RPS + i) * vdim] : 0.f;
    float* out = a.out + (long long)row0 * a.n_heads * vdim + (long long)h * vdim + col;
    const int out_step = a.n_heads * vdim;

    for (int gi = 0; gi < groups; ++gi) {
        const float* stage = dc_ring + (gi % DC_STAGES) * R::STAGE;
        dc_wait_oldest();
        __syncthreads();            // this group's record is there for every warp, and every warp is done with the one before
        const int ahead = gi + DC_STAGES - 1;
        if (ahead < groups) dc_ask<RPS>(rec0 + ahead * rec_step, vp, c0, dc_ring + (ahead % DC_STAGES) * R::STAGE, tid);
        dc_commit();
        const float* mine = stage + r * R::SLICE;
        // this lane's parts of S^T kd_t (x[t]) and S^T qd_t (x[C + t])
        float x[2 * DC_C];
#pragma unroll
        for (int t = 0; t < 2 * DC_C; ++t) {
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int i = 0; i < RPS; i += 4) {
                const float4 m = *reinterpret_cast<const float4*>(mine + t * R::VEC + i);
                acc0 = fmaf(s[i], m.x, acc0); acc1 = fmaf(s[i + 1], m.y, acc1); acc0 = fmaf(s[i + 2], m.z, acc0); acc1 = fmaf(s[i + 3], m.w, acc1);
            }
            x[t] = acc0 + acc1;
        }
        const float z = dc_sum16(x, r);
        const float* sc = stage + R::SC;
        // Lanes 0..7 of a column hold S^T kd_t, lanes 8..15 S^T qd_t.  r_t = v_t - S^T kd_t goes to every lane; lane t then
        // forms u_t = (T r)_t and lane 8 + t o_t = S^T qd_t + (B T r)_t, a row of eight products each.
        const int left = n - gi * DC_C;
        const int tt = r & 7;
        const float val = r < DC_C ? stage[R::V + tt * DC_COLS + bc] - z : z;
        float rj[DC_C];
#pragma unroll
        for (int j = 0; j < DC_C; ++j) rj[j] = __shfl_sync(full, val, j, 16);
        const float* mrow = sc + r * DC_C;            // row t of T for lanes 0..7, row t of B T for lanes 8..15
        const float4 m_lo = *reinterpret_cast<const float4*>(mrow), m_hi = *reinterpret_cast<const float4*>(mrow + 4);
        float acc = r < DC_C ? 0.f : z;
        acc = fmaf(m_lo.x, rj[0], acc); acc = fmaf(m_lo.y, rj[1], acc); acc = fmaf(m_lo.z, rj[2], acc); acc = fmaf(m_lo.w, rj[3], acc);
        acc = fmaf(m_hi.x, rj[4], acc); acc = fmaf(m_hi.y, rj[5], acc); acc = fmaf(m_hi.z, rj[6], acc); acc = fmaf(m_hi.w, rj[7], acc);
        if (r >= DC_C && col_ok && tt < left) out[(long long)(gi * DC_C + tt) * out_step] = acc;
        float u[DC_C];
#pragma unroll
        for (int j = 0; j < DC_C; ++j) u[j] = __shfl_sync(full, acc, j, 16);
        // S' = P(0, C) (.) S + sum_j w_j u_j^T
#pragma unroll
        for (int i = 0; i < RPS; i += 4) {
            const float4 pc = *reinterpret_cast<const float4*>(mine + 3 * DC_C * R::VEC + i);
            s[i] *= pc.x; s[i + 1] *= pc.y; s[i + 2] *= pc.z; s[i + 3] *= pc.w;
        }
#pragma unroll
        for (int j = 0; j < DC_C; ++j) {
#pragma unroll
            for (int i = 0; i < RPS; i += 4) {
                const float4 w4 = *reinterpret_cast<const float4*>(mine + (2 * DC_C + j) * R::VEC + i);
                s[i] = fmaf(w4.x, u[j], s[i]); s[i + 1] = fmaf(w4.y, u[j], s[i + 1]); s[i + 2] = fmaf(w4.z, u[j], s[i + 2]); s[i + 3] = fmaf(w4.w, u[j], s[i + 3]);
            }
        }
    }
    dc_wait_all();
#pragma unroll
    for (int i = 0; i < RPS; ++i)
        if (col_ok && r * RPS + i < dim) S[(long long)(r * RPS + i) * vdim] = s[i];
}

template <typename T, int RPS>
int dc_launch(const RecurrenceArgs* a, float* records, int max_groups, cudaStream_t st) {
    using R = DcRecord<RPS>;
    const size_t smem = (size_t)DC_STAGES * R::STAGE * sizeof(float);
    static bool opted = false;
    if (!opted) {
        RDL_CUDA(cudaFuncSetAttribute(dc_scan_kernel<RPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "delta_rule_chunked");
        opted = true;
    }
    RDL_CHECK_EX(rdl_launch(dc_record_kernel<T, RPS>, dim3(max_groups, a->n_heads), dim3(128), 0, st, *a, records), "delta_rule_chunked (records)");
    RDL_CHECK_EX(rdl_launch(dc_scan_kernel<RPS>, dim3(a->n_seqs, a->n_heads, (a->vdim + DC_COLS - 1) / DC_COLS), dim3(DC_THREADS), smem, st, *a,
                            (const float*)records), "delta_rule_chunked (scan)");
    return 0;
}

}  // namespace

// Bytes of the work buffer: a record per group of eight tokens and head.
extern "C" long long rdl_delta_rule_chunked_work_bytes(int n_tokens, int n_seqs, int n_heads, int dim, int vdim) {
    const long long rec = dim <= 64 ? DcRecord<4>::floats(vdim) : DcRecord<8>::floats(vdim);
    return (long long)dc_max_groups(n_tokens, n_seqs) * n_heads * rec * (long long)sizeof(float);
}

extern "C" int rdl_delta_rule_chunked(const RecurrenceArgs* a, void* work, long long work_bytes, void* stream) {
    RDL_REQUIRE(rdl_valid_dtype(a->dtype) && a->mode == RDL_REC_DELTA, "delta_rule_chunked: the delta rule only");
    RDL_REQUIRE(a->n_tokens >= 0 && a->n_seqs >= 0 && a->n_heads > 0 && a->n_key_heads > 0 && a->n_heads % a->n_key_heads == 0 && a->vdim > 0,
                "delta_rule_chunked: bad sizes");
    RDL_REQUIRE(a->dim > 0 && a->dim <= 128, "delta_rule_chunked: heads of up to 128 key channels, got %d", a->dim);
    RDL_REQUIRE(a->rows && a->q_f && a->k_f && a->g_f && a->beta_f && a->tok_pos && a->seq_start && a->slots && a->state && a->out,
                "delta_rule_chunked: missing rows, prepared vectors, batch description, state or output");
    if (a->n_tokens == 0 || a->n_seqs == 0) return 0;
    RDL_REQUIRE(work && ((uintptr_t)work & 15) == 0 && work_bytes >= rdl_delta_rule_chunked_work_bytes(a->n_tokens, a->n_seqs, a->n_heads, a->dim, a->vdim),
                "delta_rule_chunked: the work buffer is missing, not 16-byte aligned or too small");
    RDL_REQUIRE(a->n_heads <= 65535 && (a->vdim + DC_COLS - 1) / DC_COLS <= 65535, "delta_rule_chunked: too many heads or columns for one grid");
    const int max_groups = dc_max_groups(a->n_tokens, a->n_seqs);
    cudaStream_t st = (cudaStream_t)stream;
    float* records = (float*)work;
    if (a->dtype == RDL_BF16) return a->dim <= 64 ? dc_launch<__nv_bfloat16, 4>(a, records, max_groups, st) : dc_launch<__nv_bfloat16, 8>(a, records, max_groups, st);
    return a->dim <= 64 ? dc_launch<float, 4>(a, records, max_groups, st) : dc_launch<float, 8>(a, records, max_groups, st);
}
