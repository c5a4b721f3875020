// The selective state space in chunks, for many tokens in bfloat16 (the token-by-token form is recurrence.cu's).
//
// Per head h of group g, with a_t = exp(-exp(A_log[h]) dt_t) and dt_t = softplus(raw_t[h] + dt_bias[h]):
//     S_t = a_t S_(t-1) + dt_t B_t x_t^T,     y_t = S_t^T C_t + D[h] x_t.
// With chunks of 64 tokens, S the state before a chunk's first token, L its tokens, i and j places inside it and
// c_i = sum_(r <= i) log2 a_r (so that the decay from after token j to token i is 2^(c_i - c_j)):
//     y_i = sum_(j <= i) (C_i . B_j) dt_j 2^(c_i - c_j) x_j  +  2^(c_i) S^T C_i  +  D x_i
//     S'  = 2^(c_(L-1)) S + U,     U = sum_j B_j (dt_j 2^(c_(L-1) - c_j) x_j)^T.
// U needs nothing of the chunks before and y needs of them only S, so the work is parallel over chunks in three launches,
// as for the fixed decay of decay_attention.cu:
//   1. ssc_chunk_kernel<false>: a block per (chunk, head, 64 state columns): U = B^T X_w on tensor cores into a float work
//      buffer [chunk][head][state][vdim], and the chunk's whole decay c_(L-1) beside it;
//   2. ssc_scan_kernel: a thread per four state elements walks its sequence's chunks, S' = 2^c S + U in float, leaving in
//      the work buffer the state BEFORE each chunk and in the cache the state after the last;
//   3. ssc_chunk_kernel<true>: P = (C B^T) (.) dt_j 2^(c_i - c_j) below the diagonal, Y = P X + 2^(c_i) (C S) + D x.
// B, C and x are bfloat16 as the convolution left them (exact operands).  Whatever is formed in float on the way to a
// tensor-core product - the weighted x of step 1, P, and the state S - goes in as two bfloat16 terms (its rounding and
// what the rounding left), so that 16 bits of it count; every sum is float.  dt, the decays and their logarithms are float.
#include "api.h"
#include "common.cuh"
#include "launch.cuh"

namespace {

#define SSC_CHUNK 64
#define SSC_COLS 64
#define SSC_THREADS 256
#define SSC_PAD 8            // bfloat16 values between rows in shared memory: ldmatrix reads eight rows without bank conflicts

__device__ __forceinline__ uint32_t ssc_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ssc_ldm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ssc_ldm4t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ssc_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ssc_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// a pair of floats as two bfloat16 pairs: the rounding, and what it left
__device__ __forceinline__ void ssc_split(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 f = __bfloat1622float2(h);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = ssc_pack(x - f.x, y - f.y);
}
__device__ __forceinline__ float ssc_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// chunks a step can have at most (every sequence may end in a partial chunk)
static inline int ssc_max_chunks(int n_tokens, int n_seqs) {
    const int by_tokens = n_tokens / SSC_CHUNK + n_seqs;
    return by_tokens < n_tokens ? by_tokens : n_tokens;
}

// chunk number `idx` of the step -> its sequence and its first token there; false beyond the step's last chunk
__device__ __forceinline__ bool ssc_find_chunk(const RecurrenceArgs& a, int idx, int& seq, int& t0) {
    for (int s = 0; s < a.n_seqs; ++s) {
        const int n = a.seq_start[s + 1] - a.seq_start[s];
        const int nc = (n > 0 && a.tok_pos[a.seq_start[s]] >= 0) ? (n + SSC_CHUNK - 1) / SSC_CHUNK : 0;
        if (idx < nc) { seq = s; t0 = idx * SSC_CHUNK; return true; }
        idx -= nc;
    }
    return false;
}

// 64 rows of `width` bfloat16 values (a multiple of 8) from packed rows into shared memory, 16 bytes a copy; rows from L on are zeros
__device__ __forceinline__ void ssc_fill(__nv_bfloat16* dst, int dst_stride, const __nv_bfloat16* src, long long src_stride, int width, int L, int tid) {
    const int per = width >> 3;
    for (int idx = tid; idx < SSC_CHUNK * per; idx += SSC_THREADS) {
        const int j = idx / per, c = (idx - j * per) << 3;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (j < L) v = *reinterpret_cast<const uint4*>(src + (long long)j * src_stride + c);
        *reinterpret_cast<uint4*>(dst + j * dst_stride + c) = v;
    }
}

template <bool OUTPUT>
__global__ void __launch_bounds__(SSC_THREADS) ssc_chunk_kernel(RecurrenceArgs a, float* __restrict__ totals, float* __restrict__ work) {
    extern __shared__ __align__(16) unsigned char ssc_raw[];
    const int dim = a.dim, vdim = a.vdim;
    const int h = blockIdx.y, c0 = blockIdx.z * SSC_COLS;
    const int nv = min(SSC_COLS, vdim - c0);               // columns of this block (a multiple of 16)
    const int qs = dim + SSC_PAD, vs = SSC_COLS + SSC_PAD;  // row strides in shared memory, in values
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(ssc_raw);    // [64][qs]  B
    __nv_bfloat16* Vh = Ks + SSC_CHUNK * qs;                            // [64][vs]  x (OUTPUT), or the weighted x's rounding
    __nv_bfloat16* Vl = Vh + SSC_CHUNK * vs;                            // [64][vs]  what that rounding left (not OUTPUT)
    __nv_bfloat16* Qs = Vl + SSC_CHUNK * vs;                            // [64][qs]  C        OUTPUT only, like the two below
    __nv_bfloat16* Sh = Qs + SSC_CHUNK * qs;                            // [dim][vs] the state before the chunk, rounded
    __nv_bfloat16* Sl = Sh + dim * vs;                                  // [dim][vs] what the rounding left
    __shared__ float dts[SSC_CHUNK], cl[SSC_CHUNK];                     // dt_j and c_j
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    int seq, t0;
    if (!ssc_find_chunk(a, blockIdx.x, seq, t0)) return;
    const int row0 = a.seq_start[seq], n = a.seq_start[seq + 1] - row0;
    const int L = min(SSC_CHUNK, n - t0);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
    const int kh = h / (a.n_heads / a.n_key_heads);
    const int ksteps = dim >> 4, n_mt = dim >> 4, nt_count = nv >> 3;
    const __nv_bfloat16* rows = (const __nv_bfloat16*)a.rows + (long long)(row0 + t0) * a.row_stride;
    float* W = work + (((long long)blockIdx.x * a.n_heads + h) * dim) * vdim + c0;     // this chunk's U, then the state before it

    // step sizes and the running logarithm of the decay: a warp, two tokens a lane, sums in token order
    if (warp == 0) {
        const float neg_a = -expf(a.a_log[h]) * 1.4426950408889634f, bias = a.dt_bias[h];
        const __nv_bfloat16* dr = (const __nv_bfloat16*)a.dt_rows + (long long)(row0 + t0) * a.dt_stride + h;
        const int j0 = 2 * lane, j1 = j0 + 1;
        const float d0 = j0 < L ? ssc_softplus(__bfloat162float(dr[(long long)j0 * a.dt_stride]) + bias) : 0.f;
        const float d1 = j1 < L ? ssc_softplus(__bfloat162float(dr[(long long)j1 * a.dt_stride]) + bias) : 0.f;
        const float l0 = neg_a * d0, l1 = neg_a * d1;
        float run = l0 + l1;                               // inclusive sums over the lanes' pairs
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, run, off);
            if (lane >= off) run += up;
        }
        dts[j0] = d0; dts[j1] = d1;
        cl[j0] = run - l1; cl[j1] = run;
    }
    ssc_fill(Ks, qs, rows + a.k_col + kh * dim, a.row_stride, dim, L, tid);
    if (OUTPUT) {
        ssc_fill(Qs, qs, rows + a.q_col + kh * dim, a.row_stride, dim, L, tid);
        ssc_fill(Vh, vs, rows + a.v_col + h * vdim + c0, a.row_stride, nv, L, tid);
        // the state before this chunk as two bfloat16 terms
#pragma unroll 4
        for (int idx = tid; idx < dim * (nv >> 2); idx += SSC_THREADS) {
            const int r = idx / (nv >> 2), c = 4 * (idx - r * (nv >> 2));
            const float4 sv = __ldcg(reinterpret_cast<const float4*>(W + (long long)r * vdim + c));
            uint2 hi, lo;
            ssc_split(sv.x, sv.y, hi.x, lo.x);
            ssc_split(sv.z, sv.w, hi.y, lo.y);
            *reinterpret_cast<uint2*>(Sh + r * vs + c) = hi;
            *reinterpret_cast<uint2*>(Sl + r * vs + c) = lo;
        }
    }
    __syncthreads();        // dts, cl (and the tiles of OUTPUT)

    if (!OUTPUT) {
        // x_j dt_j 2^(c_(L-1) - c_j), as two terms
        const float c_end = cl[L - 1];
        for (int idx = tid; idx < SSC_CHUNK * (nv >> 1); idx += SSC_THREADS) {
            const int j = idx / (nv >> 1), c = 2 * (idx - j * (nv >> 1));
            uint32_t hi = 0u, lo = 0u;
            if (j < L) {
                const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(rows + (long long)j * a.row_stride + a.v_col + h * vdim + c0 + c));
                const float wj = dts[j] * exp2f(c_end - cl[j]);
                ssc_split(v.x * wj, v.y * wj, hi, lo);
            }
            *reinterpret_cast<uint32_t*>(Vh + j * vs + c) = hi;
            *reinterpret_cast<uint32_t*>(Vl + j * vs + c) = lo;
        }
        if (tid == 0 && blockIdx.z == 0) totals[(long long)blockIdx.x * a.n_heads + h] = c_end;
        __syncthreads();
        // ---- U = B^T X_w: rows 16 warp .. + 15 of the state are this warp's ----
        if (warp < n_mt) {
            const int m0 = warp * 16;
            float u[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) u[nt][0] = u[nt][1] = u[nt][2] = u[nt][3] = 0.f;
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                uint32_t ka[4];
                ssc_ldm4t(ka, ssc_smem(Ks + (kb * 16 + ((lane >> 4) << 3) + (lane & 7)) * qs + m0 + (((lane >> 3) & 1) << 3)));
#pragma unroll
                for (int nb = 0; nb < 4; ++nb) {
                    if (2 * nb >= nt_count) continue;
                    const int off = (kb * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * vs + nb * 16 + ((lane >> 4) << 3);
                    uint32_t bh[4], bl[4];
                    ssc_ldm4t(bh, ssc_smem(Vh + off));
                    ssc_ldm4t(bl, ssc_smem(Vl + off));
                    ssc_mma(u[2 * nb], ka, bh[0], bh[1]);
                    ssc_mma(u[2 * nb + 1], ka, bh[2], bh[3]);
                    ssc_mma(u[2 * nb], ka, bl[0], bl[1]);
                    ssc_mma(u[2 * nb + 1], ka, bl[2], bl[3]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                if (nt >= nt_count) continue;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    *reinterpret_cast<float2*>(W + (long long)(m0 + g + 8 * hh) * vdim + nt * 8 + 2 * tq) = make_float2(u[nt][2 * hh], u[nt][2 * hh + 1]);
            }
        }
        return;
    }

    // ---- P = (C B^T) (.) dt_j 2^(c_i - c_j), rows 16 rw .. + 15 ----
    // warps rw and rw + 4 share the rows 16 rw .. + 15 (each forms P for itself) and take 32 of the block's 64 columns each
    const int rw = warp & 3, cw = warp >> 2;
    const int i_hi = rw * 16 + g + 8;       // this thread's rows of the chunk: i_hi - 8 and i_hi
    uint32_t qf[8][4];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
        if (kk < ksteps) ssc_ldm4(qf[kk], ssc_smem(Qs + (rw * 16 + (lane & 15)) * qs + kk * 16 + 8 * (lane >> 4)));
    float p[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) p[nt][0] = p[nt][1] = p[nt][2] = p[nt][3] = 0.f;
#pragma unroll
    for (int np = 0; np < 4; ++np) {
        if (np > rw) continue;            // keys after this warp's last row
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            if (kk >= ksteps) continue;
            uint32_t bf[4];
            ssc_ldm4(bf, ssc_smem(Ks + (np * 16 + ((lane >> 4) << 3) + (lane & 7)) * qs + kk * 16 + (((lane >> 3) & 1) << 3)));
            ssc_mma(p[2 * np], qf[kk], bf[0], bf[1]);
            ssc_mma(p[2 * np + 1], qf[kk], bf[2], bf[3]);
        }
    }
    const float ci_lo = cl[i_hi - 8], ci_hi = cl[i_hi];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = i_hi - 8 + 8 * (e >> 1), j = nt * 8 + 2 * tq + (e & 1);
            p[nt][e] = (j <= i && i < L) ? p[nt][e] * dts[j] * exp2f(((e >> 1) ? ci_hi : ci_lo) - cl[j]) : 0.f;
        }
    }
    // ---- Y = P X + 2^(c_i) C S ----
    float o[4][4], o2[4][4];          // column tiles 4 cw .. 4 cw + 3 of the block
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) { o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f; o2[nt][0] = o2[nt][1] = o2[nt][2] = o2[nt][3] = 0.f; }
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
        if (kb > rw) continue;
        uint32_t pa[4], pb[4];
        ssc_split(p[2 * kb][0], p[2 * kb][1], pa[0], pb[0]);
        ssc_split(p[2 * kb][2], p[2 * kb][3], pa[1], pb[1]);
        ssc_split(p[2 * kb + 1][0], p[2 * kb + 1][1], pa[2], pb[2]);
        ssc_split(p[2 * kb + 1][2], p[2 * kb + 1][3], pa[3], pb[3]);
#pragma unroll
        for (int nl = 0; nl < 2; ++nl) {
            const int nb = 2 * cw + nl;
            if (2 * nb >= nt_count) continue;
            uint32_t bf[4];
            ssc_ldm4t(bf, ssc_smem(Vh + (kb * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * vs + nb * 16 + ((lane >> 4) << 3)));
            ssc_mma(o[2 * nl], pa, bf[0], bf[1]);
            ssc_mma(o[2 * nl + 1], pa, bf[2], bf[3]);
            ssc_mma(o[2 * nl], pb, bf[0], bf[1]);
            ssc_mma(o[2 * nl + 1], pb, bf[2], bf[3]);
        }
    }
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        if (kk >= ksteps) continue;
#pragma unroll
        for (int nl = 0; nl < 2; ++nl) {
            const int nb = 2 * cw + nl;
            if (2 * nb >= nt_count) continue;
            const int off = (kk * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * vs + nb * 16 + ((lane >> 4) << 3);
            uint32_t bh[4], bl[4];
            ssc_ldm4t(bh, ssc_smem(Sh + off));
            ssc_ldm4t(bl, ssc_smem(Sl + off));
            ssc_mma(o2[2 * nl], qf[kk], bh[0], bh[1]);
            ssc_mma(o2[2 * nl + 1], qf[kk], bh[2], bh[3]);
            ssc_mma(o2[2 * nl], qf[kk], bl[0], bl[1]);
            ssc_mma(o2[2 * nl + 1], qf[kk], bl[2], bl[3]);
        }
    }
    const float w_lo = exp2f(ci_lo), w_hi = exp2f(ci_hi);
    const float d_skip = a.d_skip ? a.d_skip[h] : 0.f;
    float* out_lo = a.out + (long long)(row0 + t0 + i_hi - 8) * a.n_heads * vdim + (long long)h * vdim + c0;
    float* out_hi = out_lo + 8LL * a.n_heads * vdim;
#pragma unroll
    for (int nl = 0; nl < 4; ++nl) {
        const int nt = 4 * cw + nl;
        if (nt >= nt_count) continue;
        const int c = nt * 8 + 2 * tq;
        if (i_hi - 8 < L) {
            const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Vh + (i_hi - 8) * vs + c));
            *reinterpret_cast<float2*>(out_lo + c) = make_float2(fmaf(d_skip, x.x, fmaf(w_lo, o2[nl][0], o[nl][0])), fmaf(d_skip, x.y, fmaf(w_lo, o2[nl][1], o[nl][1])));
        }
        if (i_hi < L) {
            const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Vh + i_hi * vs + c));
            *reinterpret_cast<float2*>(out_hi + c) = make_float2(fmaf(d_skip, x.x, fmaf(w_hi, o2[nl][2], o[nl][2])), fmaf(d_skip, x.y, fmaf(w_hi, o2[nl][3], o[nl][3])));
        }
    }
}

// S' = 2^c S + U over a sequence's chunks, a thread per four state elements; the work buffer keeps the state before each chunk
__global__ void __launch_bounds__(128) ssc_scan_kernel(RecurrenceArgs a, const float* __restrict__ totals, float* __restrict__ work) {
    rdl_grid_wait();
    rdl_grid_launch_dependents();
    const int seq = blockIdx.x, h = blockIdx.y;
    const int row0 = a.seq_start[seq], n = a.seq_start[seq + 1] - row0;
    if (n <= 0 || a.tok_pos[row0] < 0) return;
    int first = 0;                                  // the step's chunks before this sequence's
    for (int s = 0; s < seq; ++s) {
        const int m = a.seq_start[s + 1] - a.seq_start[s];
        if (m > 0 && a.tok_pos[a.seq_start[s]] >= 0) first += (m + SSC_CHUNK - 1) / SSC_CHUNK;
    }
    const long long per = (long long)a.dim * a.vdim;          // a multiple of 4 (both sizes are multiples of 16)
    const long long e = 4 * ((long long)blockIdx.z * blockDim.x + threadIdx.x);
    if (e >= per) return;
    float4* S = reinterpret_cast<float4*>(a.state + ((long long)a.slots[seq] * a.n_heads + h) * per + e);
    float4 s = *S;
    const int chunks = (n + SSC_CHUNK - 1) / SSC_CHUNK;
    float4* w = reinterpret_cast<float4*>(work + ((long long)first * a.n_heads + h) * per + e);
    const float* tot = totals + (long long)first * a.n_heads + h;
    const long long step = (long long)a.n_heads * per / 4;
    // four chunks' values are asked for while the four before them are summed and stored: loads stay in flight throughout
    float4 u[4], nx[4];
    float d[4], nd[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        u[i] = i < chunks ? __ldcg(w + i * step) : make_float4(0.f, 0.f, 0.f, 0.f);
        d[i] = i < chunks ? exp2f(__ldcg(tot + (long long)i * a.n_heads)) : 0.f;
    }
    for (int c = 0; c < chunks; c += 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            nx[i] = c + 4 + i < chunks ? __ldcg(w + (4 + i) * step) : make_float4(0.f, 0.f, 0.f, 0.f);
            nd[i] = c + 4 + i < chunks ? exp2f(__ldcg(tot + (long long)(c + 4 + i) * a.n_heads)) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (c + i < chunks) {
                __stcg(w + i * step, s);
                s.x = fmaf(d[i], s.x, u[i].x); s.y = fmaf(d[i], s.y, u[i].y); s.z = fmaf(d[i], s.z, u[i].z); s.w = fmaf(d[i], s.w, u[i].w);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { u[i] = nx[i]; d[i] = nd[i]; }
        w += 4 * step;
    }
    *S = s;
}

}  // namespace

// Bytes of the work buffer: the chunks' decays [chunks][heads] (padded to 16 bytes) and a state per chunk and head.
extern "C" long long rdl_state_space_chunked_work_bytes(int n_tokens, int n_seqs, int n_heads, int dim, int vdim) {
    const long long chunks = ssc_max_chunks(n_tokens, n_seqs);
    const long long totals = (chunks * n_heads + 3) / 4 * 4;
    return (totals + chunks * n_heads * dim * vdim) * (long long)sizeof(float);
}

extern "C" int rdl_state_space_chunked(const RecurrenceArgs* a, void* work, long long work_bytes, void* stream) {
    RDL_REQUIRE(a->dtype == RDL_BF16 && a->mode == RDL_REC_SSM, "state_space_chunked: bfloat16 rows of the state space form only");
    RDL_REQUIRE(a->n_tokens >= 0 && a->n_seqs >= 0 && a->n_heads > 0 && a->n_key_heads > 0 && a->n_heads % a->n_key_heads == 0,
                "state_space_chunked: bad sizes");
    RDL_REQUIRE(a->dim % 16 == 0 && a->dim >= 16 && a->dim <= 128 && a->vdim % 16 == 0 && a->vdim >= 16,
                "state_space_chunked: state size %d and head size %d must be multiples of 16, the state size at most 128", a->dim, a->vdim);
    RDL_REQUIRE(a->rows && a->dt_rows && a->dt_bias && a->a_log && a->tok_pos && a->seq_start && a->slots && a->state && a->out,
                "state_space_chunked: missing rows, step sizes, parameters, batch description, state or output");
    RDL_REQUIRE(((uintptr_t)a->rows & 15) == 0 && a->row_stride % 8 == 0 && a->q_col % 8 == 0 && a->k_col % 8 == 0 && a->v_col % 8 == 0,
                "state_space_chunked: rows and the columns of x, B and C must start on 16-byte boundaries");
    RDL_REQUIRE(((uintptr_t)a->out & 7) == 0 && ((uintptr_t)a->state & 15) == 0 && ((uintptr_t)work & 15) == 0,
                "state_space_chunked: the output must be 8-byte aligned, state and work buffer 16-byte aligned");
    if (a->n_tokens == 0 || a->n_seqs == 0) return 0;
    const int max_chunks = ssc_max_chunks(a->n_tokens, a->n_seqs);
    RDL_REQUIRE(work && work_bytes >= rdl_state_space_chunked_work_bytes(a->n_tokens, a->n_seqs, a->n_heads, a->dim, a->vdim),
                "state_space_chunked: the work buffer is too small");
    RDL_REQUIRE(a->n_heads <= 65535 && (a->vdim + SSC_COLS - 1) / SSC_COLS <= 65535, "state_space_chunked: too many heads or columns for one grid");
    float* totals = (float*)work;
    float* states = totals + ((long long)max_chunks * a->n_heads + 3) / 4 * 4;
    const int qs = a->dim + SSC_PAD, vs = SSC_COLS + SSC_PAD;
    const size_t smem_u = (size_t)(SSC_CHUNK * qs + 2 * SSC_CHUNK * vs) * 2;
    const size_t smem_o = (size_t)(2 * SSC_CHUNK * qs + 2 * SSC_CHUNK * vs + 2 * a->dim * vs) * 2;
    static bool opted = false;
    if (!opted) {
        RDL_CUDA(cudaFuncSetAttribute(ssc_chunk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024), "state_space_chunked");
        opted = true;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const dim3 grid(max_chunks, a->n_heads, (a->vdim + SSC_COLS - 1) / SSC_COLS);
    RDL_CHECK_EX(rdl_launch(ssc_chunk_kernel<false>, grid, dim3(SSC_THREADS), smem_u, st, *a, totals, states), "state_space_chunked (chunk states)");
    const long long per = (long long)a->dim * a->vdim;
    RDL_CHECK_EX(rdl_launch(ssc_scan_kernel, dim3(a->n_seqs, a->n_heads, (unsigned)((per / 4 + 127) / 128)), dim3(128), 0, st, *a, (const float*)totals, states),
                 "state_space_chunked (scan)");
    RDL_CHECK_EX(rdl_launch(ssc_chunk_kernel<true>, grid, dim3(SSC_THREADS), smem_o, st, *a, totals, states), "state_space_chunked (outputs)");
    return 0;
}
