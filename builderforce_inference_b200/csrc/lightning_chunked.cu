// Linear attention with a per-head decay over runs of new tokens, on the tensor cores: the same
// recurrence as lightning.cu (S_t = w S_(t-1) + k_t v_t^T, o_t = S_t^T q_t), evaluated a chunk of
// 64 tokens at a time.  With S the state before the chunk, t and j counted inside the chunk and n
// its length:
//     o_t  = w^(t+1) (q_t S)  +  sum_{j <= t} w^(t-j) (q_t . k_j) v_j
//     S'   = w^n S  +  sum_j w^(n-1-j) k_j v_j^T
// Only non-negative powers of w appear, so any decay in [0, 1] is safe.  q, k, v are the activated
// projections rounded to bfloat16 (products of two bfloat16 values are exact in float32); the
// state, the scores, the decayed weights and every sum are float32.  Where a float32 matrix has
// to be a tensor-core operand (S in q S, the decayed scores, the decayed values) it is split
// into a bfloat16 head and a bfloat16 remainder and the product is taken with both, which keeps
// 16 bits of mantissa; the master copy of the state stays float32 and is only ever added to.
//
// A block (16 warps) owns VB columns of one head of one sequence and walks the sequence's chunks in order;
// the matrix products are 16x16 tiles of mma.sync.m16n8k16 (operands by ldmatrix) dealt round-robin to
// its warps.
#include "attention_tiles.cuh"

#define LC 64          // tokens per chunk
#define LC_WARPS 16     // (AD_WARPS of attention_tiles.cuh belongs to the attention kernels)

__device__ __forceinline__ float lc_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

struct LcSmem {
    int ldq, ldv, lda, ldaf, ldof, ldsf;
    size_t q, k, v, af, ahi, alo, of, vhi, vlo, sf, shi, slo, pw, total;
};

static __host__ __device__ inline LcSmem lc_layout(int D, int VB) {
    LcSmem s;
    s.ldq = D + 8, s.ldv = VB + 8, s.lda = LC + 8, s.ldaf = LC + 4, s.ldof = VB + 4, s.ldsf = VB + 4;
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t at = o; o += (bytes + 127) / 128 * 128; return at; };
    s.q = take((size_t)LC * s.ldq * 2);
    s.k = take((size_t)LC * s.ldq * 2);
    s.v = take((size_t)LC * s.ldv * 2);
    s.af = take((size_t)LC * s.ldaf * 4);
    s.ahi = take((size_t)LC * s.lda * 2);
    s.alo = take((size_t)LC * s.lda * 2);
    s.of = take((size_t)LC * s.ldof * 4);
    s.vhi = take((size_t)LC * s.ldv * 2);
    s.vlo = take((size_t)LC * s.ldv * 2);
    s.sf = take((size_t)D * s.ldsf * 4);
    s.shi = take((size_t)D * s.ldv * 2);
    s.slo = take((size_t)D * s.ldv * 2);
    s.pw = take((size_t)(LC + 1) * 4);
    s.total = o;
    return s;
}

// Operands of mma.sync.m16n8k16 out of shared memory by ldmatrix, for a 16x16 tile of the result (two
// blocks of 8 columns: b[0], b[1] feed the first, b[2], b[3] the second).  "rows": the tile lies
// as it is multiplied (A as [m][k], B as [k][n]); "cols": it lies transposed (A as [k][m], B as [n][k]).
__device__ __forceinline__ void lc_a_rows(uint32_t (&a)[4], const bf16* tile, int ld) {
    const int lane = threadIdx.x & 31;
    ldmatrix_x4(a, tile + (lane & 15) * ld + (lane >> 4) * 8);
}
__device__ __forceinline__ void lc_a_cols(uint32_t (&a)[4], const bf16* tile, int ld) {
    const int lane = threadIdx.x & 31;
    ldmatrix_x4_trans(a, tile + ((lane & 7) + ((lane >> 4) << 3)) * ld + ((lane >> 3) & 1) * 8);
}
__device__ __forceinline__ void lc_b_rows(uint32_t (&b)[4], const bf16* tile, int ld) {
    const int lane = threadIdx.x & 31;
    ldmatrix_x4_trans(b, tile + (lane & 15) * ld + (lane >> 4) * 8);
}
__device__ __forceinline__ void lc_b_cols(uint32_t (&b)[4], const bf16* tile, int ld) {
    const int lane = threadIdx.x & 31;
    ldmatrix_x4(b, tile + ((lane & 7) + ((lane >> 4) << 3)) * ld + ((lane >> 3) & 1) * 8);
}
// The 16x16 float32 tile of a warp's accumulators to and from shared memory.
__device__ __forceinline__ void lc_store(float* tile, int ld, const float (&acc)[2][4]) {
    const int g = (threadIdx.x & 31) >> 2, t = threadIdx.x & 3;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
        *reinterpret_cast<float2*>(tile + g * ld + nb * 8 + 2 * t) = make_float2(acc[nb][0], acc[nb][1]);
        *reinterpret_cast<float2*>(tile + (g + 8) * ld + nb * 8 + 2 * t) = make_float2(acc[nb][2], acc[nb][3]);
    }
}
__device__ __forceinline__ void lc_load(float (&acc)[2][4], const float* tile, int ld) {
    const int g = (threadIdx.x & 31) >> 2, t = threadIdx.x & 3;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
        const float2 lo = *reinterpret_cast<const float2*>(tile + g * ld + nb * 8 + 2 * t);
        const float2 hi = *reinterpret_cast<const float2*>(tile + (g + 8) * ld + nb * 8 + 2 * t);
        acc[nb][0] = lo.x, acc[nb][1] = lo.y, acc[nb][2] = hi.x, acc[nb][3] = hi.y;
    }
}

__device__ __forceinline__ void lc_split(float x, bf16& hi, bf16& lo) {
    hi = __float2bfloat16_rn(x);
    lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

// DC: the head's dim when it is known at compile time (the products' loops over it are then unrolled
// and their operand loads run ahead of the tensor-core instructions), 0 for any multiple of 16.
template <int VB, int DC>
__global__ void __launch_bounds__(LC_WARPS * 32)
lightning_chunk_kernel(const bf16* __restrict__ proj, long stride, int q_off, int k_off, int v_off, float* __restrict__ out,
                       long out_stride, float* __restrict__ state, const float* __restrict__ decay,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slot, int H, int V,
                       int D_any, int v_blocks) {
    pdl_trigger();
    const int D = DC ? DC : D_any;
    extern __shared__ __align__(128) unsigned char lc_smem[];
    const LcSmem L = lc_layout(D, VB);
    bf16* Qs = reinterpret_cast<bf16*>(lc_smem + L.q);
    bf16* Ks = reinterpret_cast<bf16*>(lc_smem + L.k);
    bf16* Vs = reinterpret_cast<bf16*>(lc_smem + L.v);
    float* Af = reinterpret_cast<float*>(lc_smem + L.af);
    bf16* Ahi = reinterpret_cast<bf16*>(lc_smem + L.ahi);
    bf16* Alo = reinterpret_cast<bf16*>(lc_smem + L.alo);
    float* Of = reinterpret_cast<float*>(lc_smem + L.of);
    bf16* Vhi = reinterpret_cast<bf16*>(lc_smem + L.vhi);
    bf16* Vlo = reinterpret_cast<bf16*>(lc_smem + L.vlo);
    float* Sf = reinterpret_cast<float*>(lc_smem + L.sf);
    bf16* Shi = reinterpret_cast<bf16*>(lc_smem + L.shi);
    bf16* Slo = reinterpret_cast<bf16*>(lc_smem + L.slo);
    float* pw = reinterpret_cast<float*>(lc_smem + L.pw);

    const int seq = blockIdx.y;
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int h = blockIdx.x / v_blocks;
    const int v0 = (blockIdx.x - h * v_blocks) * VB;
    const int t0 = cu_seqlens[seq], nt = cu_seqlens[seq + 1] - t0;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int DT = D / 16;
    constexpr int VT = VB / 16, CT = LC / 16;
    const float w = decay[h];
    for (int p = tid; p <= LC; p += blockDim.x) pw[p] = powf(w, (float)p);
    // the state earlier steps left (zero for a fresh slot): not written by this step's kernels
    float* sp = state + (((size_t)slot * H + h) * D) * V + v0;
    for (int i = tid; i < D * VB; i += blockDim.x) {
        const int d = i / VB, c = i - d * VB;
        const float s = v0 + c < V ? sp[(size_t)d * V + c] : 0.0f;
        Sf[d * L.ldsf + c] = s;
        lc_split(s, Shi[d * L.ldv + c], Slo[d * L.ldv + c]);
    }
    pdl_wait();

    // A chunk's q, k (all of the head) and v (this block's columns) travel as 16-byte pieces: a thread
    // asks for the next chunk's pieces before it works on this one, and activates and stores them
    // when their turn comes, so the trip to memory hides behind a chunk's products.
    const int D8 = D >> 3;
    constexpr int VB8 = VB / 8;
    constexpr int NQ = LC * 16 / (LC_WARPS * 32), NV = (LC * VB8 + LC_WARPS * 32 - 1) / (LC_WARPS * 32);
    uint4 rq[NQ], rk[NQ], rv[NV];
    auto fetch = [&](int c0) {
        const int n = min(LC, nt - c0);
#pragma unroll
        for (int u = 0; u < NQ; ++u) {
            const int idx = tid + u * LC_WARPS * 32, t = idx / D8, e = idx - t * D8;
            rq[u] = rk[u] = make_uint4(0u, 0u, 0u, 0u);
            if (t < n) {
                const bf16* row = proj + (size_t)(t0 + c0 + t) * stride + (size_t)h * D + e * 8;
                rq[u] = *reinterpret_cast<const uint4*>(row + q_off);
                rk[u] = *reinterpret_cast<const uint4*>(row + k_off);
            }
        }
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int idx = tid + u * LC_WARPS * 32, t = idx / VB8, e = idx - t * VB8;
            rv[u] = make_uint4(0u, 0u, 0u, 0u);
            if (t < n)
                rv[u] = *reinterpret_cast<const uint4*>(proj + (size_t)(t0 + c0 + t) * stride + v_off + (size_t)h * V + v0 + e * 8);
        }
    };
    auto activate = [](uint4 raw) {
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
            const __nv_bfloat162 y = __floats2bfloat162_rn(lc_silu(__low2float(x)), lc_silu(__high2float(x)));
            w[j] = *reinterpret_cast<const uint32_t*>(&y);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    };
    auto stash = [&]() {
#pragma unroll
        for (int u = 0; u < NQ; ++u) {
            const int idx = tid + u * LC_WARPS * 32, t = idx / D8, e = idx - t * D8;
            if (t < LC) {
                *reinterpret_cast<uint4*>(Qs + t * L.ldq + e * 8) = activate(rq[u]);
                *reinterpret_cast<uint4*>(Ks + t * L.ldq + e * 8) = activate(rk[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < NV; ++u) {
            const int idx = tid + u * LC_WARPS * 32, t = idx / VB8, e = idx - t * VB8;
            if (t < LC) *reinterpret_cast<uint4*>(Vs + t * L.ldv + e * 8) = activate(rv[u]);
        }
    };
    fetch(0);
    stash();
    __syncthreads();

    for (int c0 = 0; c0 < nt; c0 += LC) {
        const int n = min(LC, nt - c0);
        if (c0 + LC < nt) fetch(c0 + LC);

        // ---- scores q k^T (tiles at or below the diagonal) and q S
        constexpr int n_a = CT * (CT + 1) / 2, n_o = CT * VT;
        for (int job = warp; job < n_a + n_o; job += LC_WARPS) {
            float acc[2][4] = {};
            uint32_t fa[4], fb[4];
            if (job < n_a) {
                int ti = 0, rest = job;
                while (rest > ti) rest -= ++ti;              // job -> (ti, tj) with tj <= ti
                const int tj = rest;
#pragma unroll
                for (int kk = 0; kk < (DC ? DC / 16 : DT); ++kk) {
                    lc_a_rows(fa, Qs + ti * 16 * L.ldq + kk * 16, L.ldq);
                    lc_b_cols(fb, Ks + tj * 16 * L.ldq + kk * 16, L.ldq);      // B[k = d][n = j] = k_j[d]
                    mma16816(acc[0], fa, fb[0], fb[1]);
                    mma16816(acc[1], fa, fb[2], fb[3]);
                }
                lc_store(Af + ti * 16 * L.ldaf + tj * 16, L.ldaf, acc);
            } else {
                const int ti = (job - n_a) / VT, tv = (job - n_a) - ti * VT;
#pragma unroll
                for (int kk = 0; kk < (DC ? DC / 16 : DT); ++kk) {
                    lc_a_rows(fa, Qs + ti * 16 * L.ldq + kk * 16, L.ldq);
                    lc_b_rows(fb, Shi + kk * 16 * L.ldv + tv * 16, L.ldv);
                    mma16816(acc[0], fa, fb[0], fb[1]);
                    mma16816(acc[1], fa, fb[2], fb[3]);
                    lc_b_rows(fb, Slo + kk * 16 * L.ldv + tv * 16, L.ldv);
                    mma16816(acc[0], fa, fb[0], fb[1]);
                    mma16816(acc[1], fa, fb[2], fb[3]);
                }
                lc_store(Of + ti * 16 * L.ldof + tv * 16, L.ldof, acc);
            }
        }
        __syncthreads();

        // ---- the decays, in float32: scores, the q S rows, the values for the state, the state itself
        for (int i = tid; i < LC * LC; i += blockDim.x) {
            const int t = i / LC, j = i - t * LC;
            const float x = j <= t ? pw[t - j] * Af[t * L.ldaf + j] : 0.0f;
            lc_split(x, Ahi[t * L.lda + j], Alo[t * L.lda + j]);
        }
        for (int i = tid; i < LC * VB; i += blockDim.x) {
            const int t = i / VB, c = i - t * VB;
            Of[t * L.ldof + c] *= pw[t + 1];
            const float x = t < n ? pw[n - 1 - t] * __bfloat162float(Vs[t * L.ldv + c]) : 0.0f;
            lc_split(x, Vhi[t * L.ldv + c], Vlo[t * L.ldv + c]);
        }
        for (int i = tid; i < D * VB; i += blockDim.x) {
            const int d = i / VB, c = i - d * VB;
            Sf[d * L.ldsf + c] *= pw[n];
        }
        __syncthreads();

        // ---- o += (decayed scores) v ;  S += k^T (decayed v)
        const int n_s = DT * VT;
        for (int job = warp; job < n_o + n_s; job += LC_WARPS) {
            float acc[2][4];
            uint32_t fa[4], fb[4];
            if (job < n_o) {
                const int ti = job / VT, tv = job - ti * VT;
                lc_load(acc, Of + ti * 16 * L.ldof + tv * 16, L.ldof);
#pragma unroll
                for (int kj = 0; kj < CT; ++kj) {
                    if (kj > ti) break;
                    lc_b_rows(fb, Vs + kj * 16 * L.ldv + tv * 16, L.ldv);
                    lc_a_rows(fa, Ahi + ti * 16 * L.lda + kj * 16, L.lda);
                    mma16816(acc[0], fa, fb[0], fb[1]);
                    mma16816(acc[1], fa, fb[2], fb[3]);
                    lc_a_rows(fa, Alo + ti * 16 * L.lda + kj * 16, L.lda);
                    mma16816(acc[0], fa, fb[0], fb[1]);
                    mma16816(acc[1], fa, fb[2], fb[3]);
                }
                lc_store(Of + ti * 16 * L.ldof + tv * 16, L.ldof, acc);
            } else {
                const int td = (job - n_o) / VT, tv = (job - n_o) - td * VT;
                lc_load(acc, Sf + td * 16 * L.ldsf + tv * 16, L.ldsf);
#pragma unroll
                for (int kj = 0; kj < CT; ++kj) {
                    lc_a_cols(fa, Ks + kj * 16 * L.ldq + td * 16, L.ldq);        // A[m = d][k = j] = k_j[d]
                    lc_b_rows(fb, Vhi + kj * 16 * L.ldv + tv * 16, L.ldv);
                    mma16816(acc[0], fa, fb[0], fb[1]);
                    mma16816(acc[1], fa, fb[2], fb[3]);
                    lc_b_rows(fb, Vlo + kj * 16 * L.ldv + tv * 16, L.ldv);
                    mma16816(acc[0], fa, fb[0], fb[1]);
                    mma16816(acc[1], fa, fb[2], fb[3]);
                }
                lc_store(Sf + td * 16 * L.ldsf + tv * 16, L.ldsf, acc);
            }
        }
        __syncthreads();

        // ---- the chunk's outputs, and the new state split for the next chunk
        for (int i = tid; i < n * VB; i += blockDim.x) {
            const int t = i / VB, c = i - t * VB;
            if (v0 + c < V) out[(size_t)(t0 + c0 + t) * out_stride + (size_t)h * V + v0 + c] = Of[t * L.ldof + c];
        }
        for (int i = tid; i < D * VB; i += blockDim.x) {
            const int d = i / VB, c = i - d * VB;
            lc_split(Sf[d * L.ldsf + c], Shi[d * L.ldv + c], Slo[d * L.ldv + c]);
        }
        // ... and, in the same phase, the next chunk's q, k, v (the products that read this chunk's are done)
        if (c0 + LC < nt) stash();
        __syncthreads();
    }
    for (int i = tid; i < D * VB; i += blockDim.x) {
        const int d = i / VB, c = i - d * VB;
        if (v0 + c < V) sp[(size_t)d * V + c] = Sf[d * L.ldsf + c];
    }
}

template <int VB, int DC>
static int launch_chunks(const bf16* proj, long stride, int q_off, int k_off, int v_off, float* out, long out_stride,
                         float* state, const float* decay, const int* cu_seqlens, const int* seq_slot, int n_seqs, int H,
                         int D, int V, cudaStream_t stream) {
    const LcSmem L = lc_layout(D, VB);
    const int v_blocks = (V + VB - 1) / VB;
    auto kernel = lightning_chunk_kernel<VB, DC>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total);
    if (e != cudaSuccess) return bfi_fail("lightning_chunks: cannot reserve %zu bytes of shared memory: %s", L.total, cudaGetErrorString(e));
    bfi_launch(kernel, dim3(H * v_blocks, n_seqs), dim3(LC_WARPS * 32), L.total, stream, proj, stride, q_off, k_off, v_off, out,
               out_stride, state, decay, cu_seqlens, seq_slot, H, V, D, v_blocks);
    return bfi_check_launch("lightning_chunks");
}

// Returns 2 ("not taken") for sizes this kernel does not handle; the caller then runs the general one.
extern "C" int bfi_lightning_chunks_bf16(const void* proj, long stride, int q_off, int k_off, int v_off, float* out,
                                         long out_stride, float* state, const float* decay, const int* cu_seqlens,
                                         const int* seq_slot, int n_seqs, int H, int D, int V, cudaStream_t stream) {
    BFI_REQUIRE(H > 0 && D > 0 && V > 0, "lightning_chunks: bad sizes heads=%d dim=%d vdim=%d", H, D, V);
    BFI_REQUIRE(out_stride >= (long)H * V, "lightning_chunks: output stride shorter than the heads");
    if (n_seqs <= 0) return 0;
    if (D % 16 != 0 || D > 128 || V % 16 != 0 || n_seqs > 65535) return 2;
    // q, k and v are read in 16-byte pieces
    if (((uintptr_t)proj & 15) != 0 || stride % 8 != 0 || q_off % 8 != 0 || k_off % 8 != 0 || v_off % 8 != 0) return 2;
    // Columns per block.  A chunk costs a block a fixed part (its phases' barriers and latencies) and a
    // part per column, measured at 9.2, 6.3 and 4.7 us for 64, 32 and 16 columns; a launch takes as many
    // rounds as its blocks need on the GPU's SMs (one block per SM).  The cheapest product wins.
    const size_t limit = 200 * 1024;
    const int n_sm = bfi_sm_count();
    int vb = 0;
    double best = 0.0;
    for (int c = 0; c < 3; ++c) {
        const int cand = 64 >> c;
        const double per_chunk = c == 0 ? 9.2 : (c == 1 ? 6.3 : 4.7);
        if (V % cand != 0 || lc_layout(D, cand).total > limit) continue;
        const long blocks = (long)n_seqs * H * (V / cand);
        const double cost = (double)((blocks + n_sm - 1) / n_sm) * per_chunk;
        if (vb == 0 || cost < best) vb = cand, best = cost;
    }
    if (vb == 0) return 2;
    const bf16* p = (const bf16*)proj;
#define BFI_LC(VBB, DCC) \
    return launch_chunks<VBB, DCC>(p, stride, q_off, k_off, v_off, out, out_stride, state, decay, cu_seqlens, seq_slot, n_seqs, H, D, V, stream)
#define BFI_LC_D(VBB)          \
    if (D == 128) BFI_LC(VBB, 128); \
    if (D == 64) BFI_LC(VBB, 64);   \
    BFI_LC(VBB, 0)
    if (vb == 64) { BFI_LC_D(64); }
    if (vb == 32) { BFI_LC_D(32); }
    BFI_LC_D(16);
#undef BFI_LC_D
#undef BFI_LC
}

BFI_TRACE_EXPORT(lightning_chunked)
