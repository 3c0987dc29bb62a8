// Tensor-core stages of the SSD chunked forward for sm_100a: tcgen05.mma with TMEM accumulators,
// operands brought into 128-byte-swizzled shared memory by TMA (cp.async.bulk.tensor, no multicast).
//
// Shapes served here: 16-bit inputs (bf16 / fp16), headdim 64, dstate 128, chunk 256 -- the Mamba-2
// production shape; anything else runs the general stage kernels.  Three kernels:
//
//   cb          CB[m,k] = C_m . B_k per (batch, chunk, group), one CTA per 128-row block, written as a
//               16-bit [256 x 256] matrix (lower block triangle) that all heads of the group reuse from L2.
//   chunk_state S^T[n,p] = sum_k B[k,n] (w_k x[k,p]), w_k = exp(min(dA_last - dA_k, 0)) dt_k.  B and x
//               arrive by TMA, 256 threads weight the x rows in place (fp32 math, one rounding), then one
//               thread issues 16 MMAs (M=128 over n, N=64 over p, both operands MN-major).
//   chunk_scan  per (batch, chunk, head, 128-row block):  Y1 = C . H^T (state entering the chunk),
//               Y2 = (CB o L) . X with L[m,k] = exp(min(dA_m - dA_k, 0)) dt_k [k <= m] applied in place to
//               the CB blocks as they land; out = exp(dA_m) Y1 + Y2 + D x, gated by silu(z).  Y1 and Y2
//               live in 128 TMEM columns; two CTAs share an SM so one CTA's element-wise pass overlaps
//               the other's loads and MMAs.
//
// Thread roles: the first warps own the TMEM lanes (one matrix row per thread; chunk_scan uses two
// threads per row) for the element-wise work and the epilogue; the last warp allocates TMEM and its
// lane 0 issues TMA and MMA.
// Every mbarrier wait is bounded: on expiry the kernel records a code in the status word of the
// scratch buffer, skips the dependent work and still releases its TMEM before it exits.
#include "ssd_common.cuh"
#include "tc_sm100.cuh"
#include "tensor_map.cuh"

namespace mb200 {

// ---- host: tensor maps of the 16-bit operands (SWIZZLE_128B tiles) -----------------------------------
// fmt: 1 = bfloat16, 0 = float16 (the encoding of the MMA instruction descriptor)
static bool encode_16bit(CUtensorMap *map, int fmt, const void *base, int rank, const uint64_t *dims, const uint64_t *strides_bytes,
                         const uint32_t *box)
{
    return encode_tiled(map, fmt == 1 ? MB200_BF16 : MB200_F16, base, rank, dims, strides_bytes, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

namespace {

using namespace tc;

constexpr int kQ = 256, kP = 64, kN = 128;
constexpr int kThreadsTc = 160;

// status codes written to the scratch status word
enum { kStBarB = 11, kStBarX, kStBarScaled, kStBarDone, kStBarC, kStBarG1, kStBarFull, kStBarEmpty, kStBarG2, kStSmemAlign };

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b)   // two 16-bit products, one instruction
    {
        __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t v) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&v)); }
    static __device__ __forceinline__ uint32_t pack(float a, float b)
    {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
};
template <> struct Pack2<__half> {
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b)
    {
        __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t v) { return __half22float2(*reinterpret_cast<__half2 *>(&v)); }
    static __device__ __forceinline__ uint32_t pack(float a, float b)
    {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
};
template <typename T> struct Fmt;
template <> struct Fmt<__nv_bfloat16> { static constexpr int v = 1; };
template <> struct Fmt<__half> { static constexpr int v = 0; };

__device__ __forceinline__ uint8_t *align1024(uint8_t *p)
{
    return reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}
// Barrier over the 512 element-wise threads of the state-stream kernel (named barrier 1) that also ANDs a
// predicate across them, so a bounded wait that ran out in one warp stops every warp at the same point.
__device__ __forceinline__ bool stream_barrier_and(bool p)
{
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred q, o;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred o, 1, 512, q;\n\t"
        "selp.u32 %0, 1, 0, o;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)p)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ====================================================================================== C . B^T
// grid (ngroups, nchunks * 2, batch); CTA = rows [mb*128, mb*128+128) of one chunk against B rows
// [0, (mb+1)*128).  smem: C 2 x 16 KB, B 2 x 32 KB.  TMEM: 256 columns.
template <typename T>
__global__ void __launch_bounds__(kThreadsTc) ssd_tc_cb_kernel(const __grid_constant__ CUtensorMap tm_C, const __grid_constant__ CUtensorMap tm_B,
                                                              T *cb16, int nchunks, int ngroups, int *status)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = align1024(smem_raw);
    uint8_t *Cs = sm;               // 2 boxes [128 x 64]
    uint8_t *Bs = sm + 32768;       // 2 boxes [256 x 64] (only (mb+1)*128 rows loaded)
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 32768 + 65536);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 4);
    const int g = blockIdx.x, c = blockIdx.y >> 1, mb = blockIdx.y & 1, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ncols = (mb + 1) * 128;
    // a kernel launched after this one as its programmatic dependent (the cumsum, which shares no data with it) may
    // start at once; it ends with griddepcontrol.wait, so it is not complete before this grid is
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 128) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_fence_init();
    }
    if (warp == 4) tmem_alloc(tmem_slot, 256);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (warp == 4) {
        if (lane == 0) {
            mbar_expect_tx(&bars[0], 32768 + 2 * ncols * 128);
            for (int kb = 0; kb < 2; ++kb) {
                tma_load_4d(Cs + kb * 16384, &tm_C, &bars[0], kb * 64, g, c * kQ + mb * 128, b);
                for (int r = 0; r <= mb; ++r) tma_load_4d(Bs + kb * 32768 + r * 16384, &tm_B, &bars[0], kb * 64, g, c * kQ + r * 128, b);
            }
            if (mbar_wait(&bars[0], 0, status, kStBarC)) {
                tc_fence_after_sync();
                const uint32_t idesc = instr_desc_f16(128, ncols, Fmt<T>::v, 0, 0);
                for (int kb = 0; kb < 2; ++kb)
                    for (int s = 0; s < 4; ++s)
                        mma_f16_ss(tmem, smem_desc_sw128(smem_u32(Cs + kb * 16384) + s * 32, 16, 1024),
                                   smem_desc_sw128(smem_u32(Bs + kb * 32768) + s * 32, 16, 1024), idesc, (kb | s) != 0);
            }
            mma_commit(&bars[1]);
        }
    } else {
        const bool ok = __all_sync(0xffffffffu, mbar_wait(&bars[1], 0, status, kStBarDone));   // tcgen05.ld is warp-collective
        tc_fence_after_sync();
        const int m = mb * 128 + threadIdx.x;
        T *row = cb16 + ((((int64_t)b * nchunks + c) * ngroups + g) * kQ + m) * kQ;
        if (ok) {
            for (int nb = 0; nb < ncols / 32; ++nb) {
                float v[32];
                tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + nb * 32, v);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 o;
                    o.x = Pack2<T>::pack(v[8 * q + 0], v[8 * q + 1]);
                    o.y = Pack2<T>::pack(v[8 * q + 2], v[8 * q + 3]);
                    o.z = Pack2<T>::pack(v[8 * q + 4], v[8 * q + 5]);
                    o.w = Pack2<T>::pack(v[8 * q + 6], v[8 * q + 7]);
                    *reinterpret_cast<uint4 *>(row + nb * 32 + q * 8) = o;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem, 256);
}

// ====================================================================================== chunk state
// grid (nheads, nchunks, batch), 288 threads.  smem: B 2 x 32 KB (n halves, [256 k x 64 n]), x 32 KB.
// TMEM: 64 columns.  S^T[n,p] = sum_k B[k,n] (w_k x[k,p]): the per-step weight w_k is applied to the x rows
// (half as many elements as B, and x is per head anyway), one row per thread, in place, fp32 product with
// one rounding; B is used as TMA delivered it.
constexpr int kStateThreads = 288;
template <typename T>
__global__ void __launch_bounds__(kStateThreads) ssd_tc_chunk_state_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_B,
                                                                          const float *dtb, const float *dAb, float *states, int nchunks,
                                                                          int nheads, int heads_per_group, const int32_t *seq_idx, int seqlen,
                                                                          int *status)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = align1024(smem_raw);
    uint8_t *Bs = sm;               // 2 boxes [256 x 64]
    uint8_t *xs = sm + 65536;       // [256 x 64]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 98304);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 4);
    const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
    const int g = h / heads_per_group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the row weight is requested before the set-up barrier so its latency hides behind it and the TMA loads
    float pre_dA = 0.f, pre_dt = 0.f, pre_last = 0.f;
    if (threadIdx.x < 256) {
        const float *dtc = dtb + (((int64_t)b * nheads + h) * nchunks + c) * kQ;
        const float *dAc = dAb + (((int64_t)b * nheads + h) * nchunks + c) * kQ;
        pre_last = dAc[kQ - 1];
        pre_dA = dAc[threadIdx.x];
        pre_dt = dtc[threadIdx.x];
        if (seq_idx) {      // packed sequences: only steps of the chunk's last sequence reach its end state
            const int32_t *sid = seq_idx + (int64_t)b * seqlen;
            const int t = c * kQ + threadIdx.x, t_last = min(c * kQ + kQ, seqlen) - 1;
            if (t < seqlen && sid[t] != sid[t_last]) pre_dt = 0.f;
        }
    }
    if (threadIdx.x == 256) {
        mbar_init(&bars[0], 1);      // B landed
        mbar_init(&bars[1], 1);      // x landed
        mbar_init(&bars[2], 8);      // x rows weighted: one arrival per element-wise warp
        mbar_init(&bars[3], 1);      // MMAs done
        mbar_fence_init();
    }
    if (warp == 8) tmem_alloc(tmem_slot, 64);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    if (warp == 8) {
        if (lane == 0) {
            mbar_expect_tx(&bars[1], 32768);
            tma_load_4d(xs, &tm_x, &bars[1], 0, h, c * kQ, b);
            mbar_expect_tx(&bars[0], 65536);
            tma_load_4d(Bs, &tm_B, &bars[0], 0, g, c * kQ, b);
            tma_load_4d(Bs + 32768, &tm_B, &bars[0], 64, g, c * kQ, b);
            const bool ok = mbar_wait(&bars[2], 0, status, kStBarScaled) && mbar_wait(&bars[0], 0, status, kStBarB);
            if (ok) {
                tc_fence_after_sync();
                const uint32_t idesc = instr_desc_f16(128, 64, Fmt<T>::v, 1, 1);
                for (int s = 0; s < kQ / 16; ++s)
                    mma_f16_ss(tmem, smem_desc_sw128(smem_u32(Bs) + s * 2048, 32768, 1024),
                               smem_desc_sw128(smem_u32(xs) + s * 2048, 16, 1024), idesc, s != 0);
            }
            mma_commit(&bars[3]);
        }
    } else {
        const int k = threadIdx.x;
        const float w = __expf(fminf(pre_last - pre_dA, 0.f)) * pre_dt;
        const bool ok = mbar_wait(&bars[1], 0, status, kStBarX);
        if (ok) {
            const uint32_t base = smem_u32(xs) + k * 128;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
                const uint32_t addr = base + ((ch ^ (k & 7)) << 4);
                uint4 v = lds128(addr);
                uint32_t *e = reinterpret_cast<uint32_t *>(&v);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = Pack2<T>::unpack(e[q]);
                    e[q] = Pack2<T>::pack(f.x * w, f.y * w);
                }
                sts128(addr, v);
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[2]);
        const bool done = mbar_wait(&bars[3], 0, status, kStBarDone);
        tc_fence_after_sync();
        if (__all_sync(0xffffffffu, ok && done)) {   // tcgen05.ld is warp-collective
            float *S = states + (((int64_t)b * nchunks + c) * nheads + h) * (int64_t)(kP * kN);
            const int n = (warp & 3) * 32 + lane;     // TMEM lane = state index
            const int p0 = (warp >> 2) * 32;          // which half of the head's columns this warp stores
            float v[32];
            tmem_ld32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + p0, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) S[(p0 + j) * kN + n] = v[j];
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem, 64);
}

// ====================================================================================== state stream
// Chunk states and the inter-chunk recurrence in ONE pass: grid (nheads, batch), a CTA walks the chunks of its
// (batch, head) in order, so the fp32 chunk states never leave the SM.  Per chunk c it forms
// S_c^T[n,p] = sum_k B[k,n] (w_k x[k,p]) on the tensor core exactly as the chunk-state kernel does, keeps the
// running state H in registers (thread = one state index n and 16 columns p), stores the state ENTERING chunk
// c as a 16-bit [n][p] tile (the B operand of the chunk-scan kernel's C.H product, fetched there by TMA) and
// folds H <- exp(dA_last_c) H + S_c.  After the last chunk H is the final state.
// 576 threads: warps 0-15 weight the x rows and own the running state (16 warps because this work is a chain
// of shared-memory and TMEM round trips that only more warps in flight can hide), warp 16 issues TMA loads,
// warp 17 the MMAs.  Shared memory: stages of half a chunk (B 2 x 16 KB + x 16 KB per head for 128 steps) and one
// 16 KB state tile per head; TMEM: two accumulators of 64 columns per head, so the MMAs of chunk c overlap the fold
// of chunk c-1.  A CTA serves one head or two heads of one group (template parameter HEADS): with two, the B tile
// is fetched and read by the tensor core once for both (N = 128).
constexpr int kStreamMinUnits = 74;                    // (batch, head) units from which one CTA per unit pays: half the SMs
constexpr int kStreamWarps = 16;                       // element-wise warps
constexpr int kStreamThreads = (kStreamWarps + 2) * 32;
// HEADS heads of one group per CTA share the B tile: one stage is half a chunk of B (2 x 16 KB) and of every head's
// x (16 KB each).  One head: 4 stages of 48 KB; two heads: 3 stages of 64 KB; plus one 16 KB state tile per head.
template <int HEADS> struct StreamCfg {
    static constexpr uint32_t kStage = 32768 + HEADS * 16384;
    static constexpr int kStages = HEADS == 1 ? 4 : 3;
    static constexpr uint32_t kSmem = kStages * kStage + HEADS * 16384 + 256 + 1024;
};
enum { kStStreamFull = 41, kStStreamWeighted, kStStreamEmpty, kStStreamAcc, kStStreamAccEmpty };

template <typename T, int HEADS>
__global__ void __launch_bounds__(kStreamThreads, 1)
ssd_tc_state_stream_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_B,
                           const __grid_constant__ CUtensorMap tm_Hs, const float *dtb, const float *dAb, const float *initial,
                           float *final_states, float *range_decay, float *prefix_decay, float *state_copy, float *decay_copy,
                           int store_entering, int nchunks, int nheads, int heads_per_group, int unit0, const int32_t *seq_idx, int seqlen,
                           int *status)
{
    using Cfg = StreamCfg<HEADS>;
    constexpr int NST = Cfg::kStages;
    constexpr uint32_t kStage = Cfg::kStage;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = align1024(smem_raw);
    uint8_t *tile = sm + NST * kStage;
    uint64_t *bars = reinterpret_cast<uint64_t *>(tile + HEADS * 16384);
    uint64_t *full = bars, *weighted = bars + 4, *empty = bars + 8, *acc_full = bars + 12, *acc_empty = bars + 14;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 16);
    // work unit = HEADS consecutive heads of one batch row (all of one group); units are numbered batch-major
    const int unit = unit0 + blockIdx.x, upb = nheads / HEADS;
    const int h0 = (unit % upb) * HEADS, b = unit / upb;
    const int g = h0 / heads_per_group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nstages = 2 * nchunks;
    if (threadIdx.x == kStreamWarps * 32) {
        for (int i = 0; i < NST; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&weighted[i], kStreamWarps);      // one arrival per element-wise warp
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], kStreamWarps);
        }
        mbar_fence_init();
    }
    if (warp == kStreamWarps) tmem_alloc(tmem_slot, 128 * HEADS);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == kStreamWarps) {
        // ------------------------------------------------------------------ TMA loads, up to NST stages ahead
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < nstages; ++i) {
                const int st = i % NST;
                if (i >= NST && !mbar_wait(&empty[st], ((i / NST) - 1) & 1, status, kStStreamEmpty)) break;
                uint8_t *dst = sm + st * kStage;
                const int t0 = i * 128;
                mbar_expect_tx(&full[st], kStage);
                for (int hd = 0; hd < HEADS; ++hd) tma_load_4d(dst + 32768 + hd * 16384, &tm_x, &full[st], 0, h0 + hd, t0, b);
                tma_load_4d(dst, &tm_B, &full[st], 0, g, t0, b);
                tma_load_4d(dst + 16384, &tm_B, &full[st], 64, g, t0, b);
                ++issued;
            }
            // nothing may still be landing in this CTA's shared memory when it exits
            for (int i = issued > NST ? issued - NST : 0; i < issued; ++i) mbar_wait(&full[i % NST], (i / NST) & 1, status, kStStreamFull);
        }
    } else if (warp == kStreamWarps + 1) {
        // ------------------------------------------------------------------ MMAs: S^T[n, (head, p)] += B[k, n] xw[k, (head, p)]
        if (lane == 0) {
            const uint32_t idesc = instr_desc_f16(128, 64 * HEADS, Fmt<T>::v, 1, 1);
            bool ok = true;
            for (int c = 0; c < nchunks && ok; ++c) {
                const uint32_t acc = tmem + (uint32_t)(c & 1) * 64 * HEADS;
                if (c >= 2) ok = mbar_wait(&acc_empty[c & 1], ((c >> 1) - 1) & 1, status, kStStreamAccEmpty);
                for (int half = 0; half < 2 && ok; ++half) {
                    const int i = 2 * c + half, st = i % NST;
                    ok = mbar_wait(&weighted[st], (i / NST) & 1, status, kStStreamWeighted);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t sb = smem_u32(sm + st * kStage);
                    for (int s = 0; s < 8; ++s)
                        mma_f16_ss(acc, smem_desc_sw128(sb + s * 2048, 16384, 1024), smem_desc_sw128(sb + 32768 + s * 2048, 16384, 1024),
                                   idesc, (half | s) != 0);
                    mma_commit(&empty[st]);
                }
                if (ok) mma_commit(&acc_full[c & 1]);
            }
        }
    } else {
        // ------------------------------------------------------------------ element-wise warps
        const int tid = threadIdx.x;
        // weighting: the 512 threads split into HEADS groups; a group's threads share out the 128 rows x 8 chunks
        // of its head's x tile
        constexpr int TPH = kStreamWarps * 32 / HEADS, TPR = TPH / 128, NCH = 8 / TPR;
        const int whead = tid / TPH, wt = tid % TPH;
        const int r = wt / TPR, cq = (wt % TPR) * NCH;       // my x row inside a stage and my first 16-byte chunk of it
        const int n = (warp & 3) * 32 + lane;                // TMEM lane = state index
        const int p0 = (warp >> 2) * 16;                     // my quarter of every head's columns
        const int64_t bh0 = (int64_t)b * nheads + h0;
        float H[HEADS][16];
#pragma unroll
        for (int hd = 0; hd < HEADS; ++hd)
#pragma unroll
            for (int j = 0; j < 16; ++j) H[hd][j] = initial ? initial[(bh0 + hd) * (kP * kN) + (int64_t)(p0 + j) * kN + n] : 0.f;
        // per chunk: dA and dt of my two x rows (my weighting head), and every head's dA at the end of the chunk.
        // Packed sequences: a row of another sequence than the chunk's last weighs nothing (dt = 0), and a chunk
        // whose last step belongs to another sequence than the previous chunk's carries nothing over (decay 0).
        const int32_t *sid = seq_idx ? seq_idx + (int64_t)b * seqlen : nullptr;
        auto scalars = [&](int c, float (&v)[5 + HEADS]) {
            const float *dAc = dAb + ((bh0 + whead) * nchunks + c) * kQ, *dtc = dtb + ((bh0 + whead) * nchunks + c) * kQ;
            v[0] = dAc[r]; v[1] = dtc[r]; v[2] = dAc[128 + r]; v[3] = dtc[128 + r];
#pragma unroll
            for (int hd = 0; hd < HEADS; ++hd) v[4 + hd] = dAb[((bh0 + hd) * nchunks + c) * kQ + kQ - 1];
            v[4 + HEADS] = 1.f;         // 0 when nothing carries over into the state after this chunk
            if (sid) {
                const int t_last = min(c * kQ + kQ, seqlen) - 1;
                const int s_last = sid[t_last], s_prev = c > 0 ? sid[c * kQ - 1] : 0;
                const int t0r = c * kQ + r, t1r = t0r + 128;
                if (t0r < seqlen && sid[t0r] != s_last) v[1] = 0.f;
                if (t1r < seqlen && sid[t1r] != s_last) v[3] = 0.f;
                if (s_last != s_prev) v[4 + HEADS] = 0.f;
            }
        };
        float nxt[5 + HEADS];
        scalars(0, nxt);
        float dec_prev[HEADS], dA_total[HEADS];
#pragma unroll
        for (int hd = 0; hd < HEADS; ++hd) dec_prev[hd] = 0.f, dA_total[hd] = 0.f;
        bool ok = true;
        auto fold = [&](int c) {      // H <- dec H + S_c once the MMAs of chunk c have completed
            ok = __all_sync(0xffffffffu, ok && mbar_wait(&acc_full[c & 1], (c >> 1) & 1, status, kStStreamAcc));   // tcgen05.ld is warp-collective
            if (!ok) return;
            tc_fence_after_sync();
            float v[HEADS][16];
#pragma unroll
            for (int hd = 0; hd < HEADS; ++hd)
                tmem_ld16(tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(c & 1) * 64 * HEADS + hd * 64 + p0, v[hd]);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[c & 1]);
#pragma unroll
            for (int hd = 0; hd < HEADS; ++hd)
#pragma unroll
                for (int j = 0; j < 16; ++j) H[hd][j] = fmaf(dec_prev[hd], H[hd][j], v[hd][j]);
        };
        for (int c = 0; c < nchunks && ok; ++c) {
            float cur[5 + HEADS];
#pragma unroll
            for (int q = 0; q < 5 + HEADS; ++q) cur[q] = nxt[q];
            if (c + 1 < nchunks) scalars(c + 1, nxt);
            float my_last = cur[4];
#pragma unroll
            for (int hd = 1; hd < HEADS; ++hd) my_last = whead == hd ? cur[4 + hd] : my_last;
            // weight my x rows of both halves: w_k = exp(dA_last - dA_k) dt_k
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int i = 2 * c + half, st = i % NST;
                const float w = __expf(fminf(my_last - cur[2 * half], 0.f)) * cur[2 * half + 1];
                ok = ok && mbar_wait(&full[st], (i / NST) & 1, status, kStStreamFull);
                if (ok) {
                    const uint32_t base = smem_u32(sm + st * kStage + 32768 + whead * 16384) + r * 128;
#pragma unroll
                    for (int ch = 0; ch < NCH; ++ch) {
                        const uint32_t addr = base + (((cq + ch) ^ (r & 7)) << 4);
                        uint4 v = lds128(addr);
                        uint32_t *e = reinterpret_cast<uint32_t *>(&v);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float2 f = Pack2<T>::unpack(e[q]);
                            e[q] = Pack2<T>::pack(f.x * w, f.y * w);
                        }
                        sts128(addr, v);
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&weighted[st]);
            }
            if (c > 0) fold(c - 1);
#pragma unroll
            for (int hd = 0; hd < HEADS; ++hd) {
                dec_prev[hd] = __expf(cur[4 + hd]) * cur[4 + HEADS];
                if (tid == 0 && prefix_decay) prefix_decay[(bh0 + hd) * nchunks + c] = __expf(dA_total[hd]);   // decay from the range start to chunk c
                dA_total[hd] += cur[4 + hd];
            }
            // the states entering chunk c leave as 16-bit [n][p] tiles (not when only the range summary is wanted)
            if (tid == 0 && store_entering) tma_store_wait_read();   // the previous stores have finished reading the tiles
            ok = stream_barrier_and(ok);                     // from here on every element-wise warp agrees on ok
            if (!ok) break;
            if (store_entering) {
#pragma unroll
                for (int hd = 0; hd < HEADS; ++hd) {
                    const uint32_t row = smem_u32(tile + hd * 16384) + n * 128;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        uint4 o;
                        o.x = Pack2<T>::pack(H[hd][8 * q + 0], H[hd][8 * q + 1]);
                        o.y = Pack2<T>::pack(H[hd][8 * q + 2], H[hd][8 * q + 3]);
                        o.z = Pack2<T>::pack(H[hd][8 * q + 4], H[hd][8 * q + 5]);
                        o.w = Pack2<T>::pack(H[hd][8 * q + 6], H[hd][8 * q + 7]);
                        sts128(row + ((((p0 >> 3) + q) ^ (n & 7)) << 4), o);
                    }
                }
                fence_proxy_async();
                asm volatile("bar.sync 1, 512;" ::: "memory");
                if (tid == 0) {
                    for (int hd = 0; hd < HEADS; ++hd)
                        tma_store_3d(&tm_Hs, tile + hd * 16384, 0, 0, (int)((((int64_t)b * nchunks + c) * nheads) + h0 + hd));
                    tma_store_commit();
                }
            }
        }
        if (ok) fold(nchunks - 1);
#pragma unroll
        for (int hd = 0; hd < HEADS; ++hd) {
            if (ok && final_states) {
                float *F = final_states + (bh0 + hd) * (kP * kN);
#pragma unroll
                for (int j = 0; j < 16; ++j) F[(p0 + j) * kN + n] = H[hd][j];
            }
            if (ok && state_copy) {
                float *F = state_copy + (bh0 + hd) * (kP * kN);
#pragma unroll
                for (int j = 0; j < 16; ++j) F[(p0 + j) * kN + n] = H[hd][j];
            }
        }
        if (tid == 0) {
            tma_store_wait_read();
            for (int hd = 0; hd < HEADS; ++hd) {
                if (ok && range_decay) range_decay[bh0 + hd] = __expf(dA_total[hd]);
                if (ok && decay_copy) decay_copy[bh0 + hd] = __expf(dA_total[hd]);
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kStreamWarps) tmem_dealloc(tmem, 128 * HEADS);
}

// ====================================================================================== chunk scan
// grid (nheads, nchunks * 2, batch), 288 threads: warps 0-7 element-wise + epilogue (thread = one row and one
// 32-column half), warp 8 TMA + MMA.  Shared memory (74.7 KB, three CTAs per SM) is a ring of three 24 KB slots,
// each a 16 KB tile followed by 8 KB: a K half of C [128 x 64] with the matching half of the entering state H, or
// a "block" = 64-wide slice of the mask product (CB tile [128 x 64] with the 64 rows of x it multiplies).
//   C/H half 0 -> slot 0, C/H half 1 -> slot 1, block j -> slot (2 + j) % 3
// Both C/H halves and block 0 are requested at once; a slot is re-used as soon as the MMAs that read it have
// completed (block 1 after the first half of C.H^T, block 2 after its second, block 3 after block 0).  The gate tile z
// lands in the tile part of a slot that is done with (slot 1 for the first row block, slot 0 for the second);
// the output tile is assembled in the tile part of block 0's / block 2's slot and leaves through one TMA store.
// The row block's own x rows (for D x) are the x parts of its last two blocks, which nothing overwrites.
// Then scalars (dA*log2e and the column factors in fp32, dt in bf16) and barriers.
// The 16 KB tiles are never multiplied from shared memory: the element-wise threads read their 32 columns of a
// row, apply their factors (exp(dA_m) for a C half, the decay mask for a CB tile) and write 16 packed words to
// their lane of tensor memory; tcgen05.mma takes A from there and B (H half, x rows) from shared memory.
// TMEM: 128 columns = one 64-column accumulator Y for all products + two 32-column A buffers used alternately.
//
// Decay mask.  A thread owns 32 consecutive columns k of one row m per block.  Three cases:
//   all k > m           zeros
//   all k <= m          L[m,k] = exp(dA_m - dA_ref) * (exp(dA_ref - dA_k) dt_k), ref = last k of the range: one
//                       exponential per thread, the column factors are computed once per CTA.  Both exponents
//                       are <= 0 because dA_cumsum is non-increasing (A <= 0, dt >= 0); a chunk where that does
//                       not hold is detected and sent down the exact path.
//   range holds k = m   the same split with the columns past the diagonal zeroed while the range's decay span is
//                       moderate (row factor >= 1, at most 2^kMaxDiagSpan); otherwise element by element:
//                       exp(min(dA_m - dA_k, 0)) dt_k [k <= m]
// The mask factors are rounded to the input dtype and applied with packed 16-bit multiplies (two roundings
// per element instead of one; far inside the 16-bit tolerance, and it halves the instruction count).
// Largest decay span (in powers of two) of a 32-column range for which the diagonal range may use the factorised
// mask: the row factor 2^span and the smallest column factor 2^-span * dt stay far inside the fp32 range.
constexpr float kMaxDiagSpan = 80.f;
constexpr int kScanThreads = 288;
constexpr uint32_t kScanSmem = 49152 + 24576 + 1024 + 1024 + 512 + 64 + 128 + 16;   // 76496 B, base must be 1 KB aligned
__device__ __forceinline__ void scan_compute_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <typename T>
__global__ void __launch_bounds__(kScanThreads, 3)
ssd_tc_chunk_scan_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_C,
                         const __grid_constant__ CUtensorMap tm_H, const __grid_constant__ CUtensorMap tm_CB,
                         const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_out, const mb200_ssd_args a,
                         const float *dtb, const float *dAb, int nchunks, int h_np, const uint8_t *seq_start, const uint8_t *seq_carry,
                         int *status)
{
    extern __shared__ __align__(1024) uint8_t sm[];
    constexpr uint32_t kSlot = 24576, kSlotX = 16384;   // a slot: 16 KB tile (C half or CB block), then 8 KB (H half or 64 rows of x)
    float *dA2 = reinterpret_cast<float *>(sm + 73728);             // 256: dA_cumsum * log2(e)
    float *cks = dA2 + 256;                                         // 256: exp(dA_ref(k) - dA_k) dt_k, ref(k) = k | 31
    __nv_bfloat16 *dts = reinterpret_cast<__nv_bfloat16 *>(cks + 256);   // 256: dt (only the exact path reads it)
    int *mono = reinterpret_cast<int *>(sm + 73728 + 2560);         // 1 while dA_cumsum is non-increasing over the chunk
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 73728 + 2560 + 16);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 22);
    uint64_t *bar_chfull = &bars[0], *bar_z = &bars[2], *bar_g2 = &bars[3];     // bar_chfull[kb]: C / H half kb has landed
    uint64_t *bar_full = &bars[4], *bar_scaled = &bars[8], *bar_e = &bars[12];   // bar_e[j]: block j has been multiplied
    uint64_t *bar_chdone = &bars[14];                                            // bar_chdone[kb]: C.H^T part kb has been multiplied
    uint64_t *bar_chscaled = &bars[16];                                          // bar_chscaled[kb]: scaled C half kb is in tensor memory

    const int h = blockIdx.x, c = blockIdx.y >> 1, mb = blockIdx.y & 1, b = blockIdx.z;
    const int g = h / (a.nheads / a.ngroups);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = (mb + 1) * 2;   // 64-wide blocks this row block needs
    // ring of three slots: C/H half 0 -> 0, C/H half 1 -> 1, mask block j -> (2 + j) % 3
    auto slot_ptr = [&](int j) -> uint8_t * { return sm + ((2 + j) % 3) * kSlot; };
    uint8_t *ztile = mb ? sm : sm + kSlot;                // slot 0 after block 1 (second row block), slot 1 after C/H half 1 (first)
    uint8_t *otile = mb ? sm + kSlot : sm + 2 * kSlot;    // tile part of block 2's / block 0's slot, multiplied long before
    // chunk scalars are requested before the set-up barrier so their latency hides behind it
    const float *dtc = dtb + (((int64_t)b * a.nheads + h) * nchunks + c) * kQ;
    const float *dAc = dAb + (((int64_t)b * a.nheads + h) * nchunks + c) * kQ;
    float pre_dk = 0.f, pre_tk = 0.f, pre_ref = 0.f, pre_prev = 0.f;
    // Packed sequences: `lo` = first column of my row's sequence inside the chunk (columns before it belong to other
    // sequences and are masked like the columns past the diagonal); `carry` = my row continues the sequence that
    // ended the previous chunk, so the state entering the chunk reaches it.
    int lo = 0;
    bool carry = true;
    if (threadIdx.x < 256) {
        const int k = threadIdx.x;
        if (seq_start) {
            const int64_t bc = (int64_t)b * nchunks + c;
            lo = seq_start[bc * kQ + mb * 128 + (k & 127)];
            carry = lo == 0 && seq_carry[bc] != 0;
        }
        pre_dk = dAc[k];
        pre_tk = dtc[k];
        pre_ref = dAc[k | 31];
        pre_prev = k > 0 ? dAc[k - 1] : pre_dk;
    }
    if (threadIdx.x == 256) {
        mbar_init(&bar_chfull[0], 1);
        mbar_init(&bar_chfull[1], 1);
        mbar_init(&bar_chdone[0], 1);
        mbar_init(&bar_chdone[1], 1);
        mbar_init(&bar_chscaled[0], 8);
        mbar_init(&bar_chscaled[1], 8);
        mbar_init(bar_z, 1);
        mbar_init(bar_g2, 1);
        for (int i = 0; i < 4; ++i) {
            mbar_init(&bar_full[i], 1);
            mbar_init(&bar_scaled[i], 8);      // one arrival per element-wise warp
        }
        mbar_init(&bar_e[0], 1);
        mbar_init(&bar_e[1], 1);
        *mono = 1;
        mbar_fence_init();
        if (smem_u32(sm) & 1023u) atomicCAS(status, 0, kStSmemAlign);   // the swizzled tiles assume a 1 KB aligned base
    }
    if (warp == 8) tmem_alloc(tmem_slot, 128);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const int64_t unit_h = ((int64_t)b * nchunks + c) * a.nheads + h;
    const int64_t unit_g = ((int64_t)b * nchunks + c) * a.ngroups + g;

    if (warp == 8) {
        if (lane == 0) {
            bool ok = (smem_u32(sm) & 1023u) == 0;
            auto load_block = [&](int j) {
                mbar_expect_tx(&bar_full[j], 16384 + 8192);
                tma_load_3d(slot_ptr(j), &tm_CB, &bar_full[j], j * 64, mb * 128, (int)unit_g);
                tma_load_4d(slot_ptr(j) + kSlotX, &tm_x, &bar_full[j], 0, h, c * kQ + j * 64, b);
            };
            const uint32_t idesc2 = instr_desc_f16(128, 64, Fmt<T>::v, 0, 1);
            auto gemm2_block = [&](int j) {      // Y += (CB o L)_j . X_j once the element-wise warps have put the scaled tile in TMEM
                ok = ok && mbar_wait(&bar_scaled[j], 0, status, kStBarScaled);
                if (ok) {
                    tc_fence_after_sync();
                    const uint32_t sb = smem_u32(slot_ptr(j));
                    for (int s = 0; s < 4; ++s)
                        mma_f16_ts(tmem, tmem + 64 + (j & 1) * 32 + s * 8, smem_desc_sw128(sb + kSlotX + s * 2048, 16, 1024), idesc2, true);
                }
            };
            auto load_z = [&]() {
                mbar_expect_tx(bar_z, 16384);
                tma_load_4d(ztile, &tm_z, bar_z, 0, h, c * kQ + mb * 128, b);
            };
            // Everything the three slots can hold is requested at once: both C/H halves and the first mask block.
            // A slot is re-used as soon as the MMAs that read it have completed, so a row block needs two round
            // trips to memory back to back instead of three.
            auto load_ch = [&](int kb) {
                uint8_t *dst = sm + kb * kSlot;
                mbar_expect_tx(&bar_chfull[kb], 16384 + 8192);
                tma_load_4d(dst, &tm_C, &bar_chfull[kb], kb * 64, g, c * kQ + mb * 128, b);
                if (h_np) tma_load_3d(dst + kSlotX, &tm_H, &bar_chfull[kb], 0, kb * 64, (int)unit_h);   // rows n of the [n][p] state
                else tma_load_3d(dst + kSlotX, &tm_H, &bar_chfull[kb], kb * 64, 0, (int)unit_h);        // columns n of the [p][n] state
            };
            if (ok) {
                load_block(0);
                load_ch(0);
                load_ch(1);
                // the later x rows and the gate tile cannot be requested yet: have them brought into L2 now
                for (int j = 1; j < nk; ++j) tma_prefetch_l2_4d(&tm_x, 0, h, c * kQ + j * 64, b);
                if (a.z) tma_prefetch_l2_4d(&tm_z, 0, h, c * kQ + mb * 128, b);
            }
            // Y = (exp(dA_m) C) . H^T in two K halves; the row-scaled C half comes from tensor memory
            const uint32_t idesc1 = instr_desc_f16(128, 64, Fmt<T>::v, 0, h_np ? 1 : 0);
            for (int kb = 0; kb < 2; ++kb) {
                ok = ok && mbar_wait(&bar_chscaled[kb], 0, status, kStBarC);
                if (ok) {
                    tc_fence_after_sync();
                    const uint32_t hb_ = smem_u32(sm + kb * kSlot) + kSlotX;
                    for (int s = 0; s < 4; ++s)
                        mma_f16_ts(tmem, tmem + 64 + kb * 32 + s * 8,
                                   h_np ? smem_desc_sw128(hb_ + s * 2048, 16, 1024) : smem_desc_sw128(hb_ + s * 32, 16, 1024), idesc1,
                                   (kb | s) != 0);
                }
                mma_commit(&bar_chdone[kb]);
            }
            ok = ok && mbar_wait(&bar_chdone[0], 0, status, kStBarG1);
            if (ok) load_block(1);                       // slot 0
            ok = ok && mbar_wait(&bar_chdone[1], 0, status, kStBarG1);
            if (ok) {
                if (nk > 2) load_block(2);               // slot 1
                else if (a.z) load_z();
            }
            gemm2_block(0);
            if (nk > 2) {
                mma_commit(&bar_e[0]);
                ok = ok && mbar_wait(&bar_e[0], 0, status, kStBarEmpty);    // slot 2 has been read
                if (ok) load_block(3);
            }
            gemm2_block(1);
            if (nk > 2) {
                mma_commit(&bar_e[1]);                   // frees slot 0 and the second TMEM tile buffer
                if (a.z) {
                    ok = ok && mbar_wait(&bar_e[1], 0, status, kStBarEmpty);
                    if (ok) load_z();
                }
                gemm2_block(2);
                gemm2_block(3);
            }
            mma_commit(bar_g2);
        }
    } else {
        const int r = threadIdx.x & 127;    // row inside the block = TMEM lane
        const int kh = threadIdx.x >> 7;    // which 32-column half of every 64-wide block
        const int m = mb * 128 + r;         // row inside the chunk
        {
            const int k = threadIdx.x;
            dA2[k] = pre_dk * kLog2e;
            dts[k] = __float2bfloat16_rn(pre_tk);
            cks[k] = __expf(pre_ref - pre_dk) * pre_tk;
            if (pre_dk > pre_prev) *mono = 0;
        }
        const int t = c * kQ + m;
        const bool live = t < a.seqlen;     // rows past the end of the sequence compute garbage that the tile store clips
        const float Dh = (a.D && !a.D_has_hdim) ? a.D[h] : 0.f;
        scan_compute_sync();
        const float dAm = dA2[m];
        const bool factor_ok = *mono != 0;
        bool ok = (smem_u32(sm) & 1023u) == 0;
        const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);      // my row of tensor memory
        // The A operands of all products go to the tensor core through tensor memory: a thread reads its 32
        // columns of the 16 KB tile from shared memory, applies its factors, and writes 16 packed words to its TMEM
        // lane (two tile buffers of 32 columns, used alternately by the ring items).
        // First the two K halves of C, row-scaled by exp(dA_m), so that C.H^T lands in the same accumulator.
        {
            const float rs = carry ? ex2(dAm) : 0.f;
            const uint32_t rs2 = Pack2<T>::pack(rs, rs);
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
                ok = __all_sync(0xffffffffu, ok && mbar_wait(&bar_chfull[kb], 0, status, kStBarC));
                if (ok) {
                    const uint32_t rowaddr = smem_u32(sm + kb * kSlot) + r * 128;
                    uint32_t w[16];
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        const uint4 v = lds128(rowaddr + (((kh * 4 + ch) ^ (r & 7)) << 4));
                        w[4 * ch] = Pack2<T>::mul(v.x, rs2);
                        w[4 * ch + 1] = Pack2<T>::mul(v.y, rs2);
                        w[4 * ch + 2] = Pack2<T>::mul(v.z, rs2);
                        w[4 * ch + 3] = Pack2<T>::mul(v.w, rs2);
                    }
                    tmem_st16(tlane + 64 + kb * 32 + kh * 16, w);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&bar_chscaled[kb]);
            }
        }
        for (int j = 0; j < nk; ++j) {
            const int klo = j * 64 + kh * 32;       // first column of this thread's range
            ok = ok && mbar_wait(&bar_full[j], 0, status, kStBarFull);
            // the tile buffer this block goes to was last read by the product two ring items earlier
            ok = ok && mbar_wait(j < 2 ? &bar_chdone[j] : &bar_e[j - 2], 0, status, kStBarEmpty);
            ok = __all_sync(0xffffffffu, ok);       // tcgen05.st is warp-collective
            const uint32_t rowaddr = smem_u32(slot_ptr(j)) + r * 128;
            if (ok) {
                tc_fence_after_sync();
                uint32_t w[16];
                if (klo > m || klo + 31 < lo) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) w[i] = 0u;
                } else if (klo >= lo && klo + 31 <= m && factor_ok) {
                    const float rm = ex2(dAm - dA2[klo + 31]);
                    const uint64_t rm2 = pack2(rm, rm);
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        const uint4 v = lds128(rowaddr + (((kh * 4 + ch) ^ (r & 7)) << 4));
                        const uint32_t e[4] = {v.x, v.y, v.z, v.w};
                        const ulonglong2 *ck = reinterpret_cast<const ulonglong2 *>(cks + klo + ch * 8);
                        const ulonglong2 c01 = ck[0], c23 = ck[1];
                        const uint64_t cp[4] = {c01.x, c01.y, c23.x, c23.y};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            float l0, l1;
                            unpack2(mul2(rm2, cp[q]), l0, l1);
                            w[4 * ch + q] = Pack2<T>::mul(e[q], Pack2<T>::pack(l0, l1));
                        }
                    }
                } else if (klo >= lo && factor_ok && dA2[klo] - dA2[klo + 31] <= kMaxDiagSpan) {
                    // the range holds the diagonal but its decay span is moderate: same split with ref = last column
                    // (the row factor is then >= 1, bounded by 2^kMaxDiagSpan), columns past the diagonal masked
                    const float rm = ex2(dAm - dA2[klo + 31]);
                    const uint64_t rm2 = pack2(rm, rm);
                    const int dm = m - klo;             // columns 0..dm of the range are at or before the diagonal
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        const uint4 v = lds128(rowaddr + (((kh * 4 + ch) ^ (r & 7)) << 4));
                        const uint32_t e[4] = {v.x, v.y, v.z, v.w};
                        const ulonglong2 *ck = reinterpret_cast<const ulonglong2 *>(cks + klo + ch * 8);
                        const ulonglong2 c01 = ck[0], c23 = ck[1];
                        const uint64_t cp[4] = {c01.x, c01.y, c23.x, c23.y};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            float l0, l1;
                            unpack2(mul2(rm2, cp[q]), l0, l1);
                            l0 = (ch * 8 + 2 * q <= dm) ? l0 : 0.f;
                            l1 = (ch * 8 + 2 * q + 1 <= dm) ? l1 : 0.f;
                            w[4 * ch + q] = Pack2<T>::mul(e[q], Pack2<T>::pack(l0, l1));
                        }
                    }
                } else {
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        const uint4 v = lds128(rowaddr + (((kh * 4 + ch) ^ (r & 7)) << 4));
                        const uint32_t e[4] = {v.x, v.y, v.z, v.w};
                        const int kc = klo + ch * 8;
                        const float4 d0 = *reinterpret_cast<const float4 *>(dA2 + kc), d1 = *reinterpret_cast<const float4 *>(dA2 + kc + 4);
                        const uint4 tv = *reinterpret_cast<const uint4 *>(dts + kc);
                        const uint32_t *tw = reinterpret_cast<const uint32_t *>(&tv);
                        const float dk[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float2 tk = Pack2<__nv_bfloat16>::unpack(tw[q]);
                            const float l0 = (kc + 2 * q <= m && kc + 2 * q >= lo) ? ex2(fminf(dAm - dk[2 * q], 0.f)) * tk.x : 0.f;
                            const float l1 = (kc + 2 * q + 1 <= m && kc + 2 * q + 1 >= lo) ? ex2(fminf(dAm - dk[2 * q + 1], 0.f)) * tk.y : 0.f;
                            w[4 * ch + q] = Pack2<T>::mul(e[q], Pack2<T>::pack(l0, l1));
                        }
                    }
                }
                // tcgen05.st is warp-collective (.sync.aligned): it must stay here, after the per-lane mask branches
                // above have reconverged -- the lanes of a warp that holds the diagonal take different branches
                __syncwarp();
                tmem_st16(tlane + 64 + (j & 1) * 32 + kh * 16, w);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&bar_scaled[j]);
        }
        ok = ok && mbar_wait(bar_g2, 0, status, kStBarG2);
        if (a.z) ok = ok && mbar_wait(bar_z, 0, status, kStBarX);
        ok = __all_sync(0xffffffffu, ok);   // tcgen05.ld is warp-collective: the whole warp takes one path
        tc_fence_after_sync();
        if (ok) {
            float acc[32];
            tmem_ld32(tlane + kh * 32, acc);
            // row m of x sits in the x part of the slot that carried block m / 64
            const uint32_t xrow = smem_u32(slot_ptr(m >> 6) + kSlotX) + (m & 63) * 128;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int p0 = kh * 32 + q4 * 8;   // column inside the head
                const uint32_t swz = (uint32_t)(((p0 >> 3) ^ (r & 7)) << 4);
                float y[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) y[i] = acc[q4 * 8 + i];
                if (a.D) {
                    const uint4 xv = lds128(xrow + swz);
                    const uint32_t *xe = reinterpret_cast<const uint32_t *>(&xv);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 f = Pack2<T>::unpack(xe[q]);
                        const float D0 = a.D_has_hdim ? a.D[h * kP + p0 + 2 * q] : Dh;
                        const float D1 = a.D_has_hdim ? a.D[h * kP + p0 + 2 * q + 1] : Dh;
                        y[2 * q] = fmaf(f.x, D0, y[2 * q]);
                        y[2 * q + 1] = fmaf(f.y, D1, y[2 * q + 1]);
                    }
                }
                if (a.z) {
                    const uint4 zv = lds128(smem_u32(ztile) + r * 128 + swz);
                    const uint32_t *ze = reinterpret_cast<const uint32_t *>(&zv);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float2 f = Pack2<T>::unpack(ze[q]);
                        if constexpr (Fmt<T>::v == 1) {     // bfloat16 output: one MUFU per gate value is accurate enough
                            y[2 * q] *= silu_for_bf16(f.x);
                            y[2 * q + 1] *= silu_for_bf16(f.y);
                        } else {
                            y[2 * q] *= fast_silu(f.x);
                            y[2 * q + 1] *= fast_silu(f.y);
                        }
                    }
                }
                uint4 o;
                o.x = Pack2<T>::pack(y[0], y[1]);
                o.y = Pack2<T>::pack(y[2], y[3]);
                o.z = Pack2<T>::pack(y[4], y[5]);
                o.w = Pack2<T>::pack(y[6], y[7]);
                sts128(smem_u32(otile) + r * 128 + swz, o);
            }
        }
        fence_proxy_async();
        scan_compute_sync();
        if (threadIdx.x == 0 && ok && live) {      // thread 0 owns the block's first row: a block wholly past the end stores nothing
            tma_store_4d(&tm_out, otile, 0, h, c * kQ + mb * 128, b);
            tma_store_commit_and_wait_read();
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem, 128);
}

// ====================================================================================== incoming state
// Sequence split, OUTPUT half: the LOCAL half stored the entering states of the range as if nothing came in.
// Adds prefix_decay[c] * S_in to each of them (16-bit [n][p] tiles) and forms the range's end state
// range_decay * S_in + S_local.  grid (ceil(nchunks / kFixChunks), nheads, batch), 256 threads; the incoming
// state of the (batch, head) is transposed once into shared memory.  Chunks whose share has decayed to nothing
// are left alone, which for fast-decaying heads is all but the first few.
constexpr int kFixChunks = 8;
template <typename T>
__global__ void __launch_bounds__(256) ssd_incoming_state_kernel(T *prev16, const float *s_in, const float *prefix_decay, const float *s_local,
                                                                  const float *range_decay, float *final_states, int nchunks, int nheads)
{
    __shared__ float sin_np[kN * (kP + 1)];      // [n][p], padded
    __shared__ float wmax[8];
    const int h = blockIdx.y, b = blockIdx.z;
    const int64_t bh = (int64_t)b * nheads + h;
    const float *src = s_in + bh * (kP * kN);
    if (blockIdx.x > 0 && prefix_decay[bh * nchunks + blockIdx.x * kFixChunks] == 0.f) return;   // decayed to zero before this CTA's chunks
    float amax = 0.f;
    for (int e = threadIdx.x; e < kP * kN; e += 256) {
        const float v = src[e];
        sin_np[(e % kN) * (kP + 1) + e / kN] = v;    // src is [p][n]
        amax = fmaxf(amax, fabsf(v));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
    if (blockIdx.x == 0 && final_states) {
        const float d = range_decay[bh];
        for (int e = threadIdx.x; e < kP * kN; e += 256) final_states[bh * (kP * kN) + e] = fmaf(d, src[e], s_local[bh * (kP * kN) + e]);
    }
    __syncthreads();
    float smax = wmax[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) smax = fmaxf(smax, wmax[i]);
    const int c0 = blockIdx.x * kFixChunks;
    for (int c = c0; c < min(c0 + kFixChunks, nchunks); ++c) {
        const float pd = prefix_decay[bh * nchunks + c];
        // the prefix decay only shrinks along the range: once the whole share is below the smallest normal number
        // nothing is left to add (infinities and NaNs in S_in still go through)
        if (pd * smax < 1.1754944e-38f) break;
        T *tile = prev16 + (((int64_t)b * nchunks + c) * nheads + h) * (kP * kN);
        for (int v = threadIdx.x; v < kP * kN / 8; v += 256) {      // 8 consecutive p of one n per step
            const int n = v / (kP / 8), p = (v % (kP / 8)) * 8;
            uint4 raw = *reinterpret_cast<const uint4 *>(tile + n * kP + p);
            uint32_t *w = reinterpret_cast<uint32_t *>(&raw);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 f = Pack2<T>::unpack(w[q]);
                w[q] = Pack2<T>::pack(fmaf(pd, sin_np[n * (kP + 1) + p + 2 * q], f.x), fmaf(pd, sin_np[n * (kP + 1) + p + 2 * q + 1], f.y));
            }
            *reinterpret_cast<uint4 *>(tile + n * kP + p) = raw;
        }
    }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
bool mult8(const int64_t *s, int n)
{
    for (int i = 0; i < n; ++i)
        if (s[i] % 8) return false;
    return true;
}

struct TcMaps {
    CUtensorMap x, B, C, H, CB;
};

template <typename T>
int run_tc(const mb200_ssd_args &a, const SsdScratch &lay, int stage, bool h_np, cudaStream_t stream, int parts = 3)
{
    char *base = static_cast<char *>(a.scratch);
    float *dtb = reinterpret_cast<float *>(base + lay.off_dt);
    float *dAb = reinterpret_cast<float *>(base + lay.off_dA);
    float *states = reinterpret_cast<float *>(base + lay.off_states);
    T *cb16 = reinterpret_cast<T *>(base + lay.off_cb);
    T *prev16 = reinterpret_cast<T *>(base + lay.off_prev16);
    int *status = reinterpret_cast<int *>(base + lay.off_status);
    const int nc = lay.nchunks, fmt = Fmt<T>::v;
    const uint64_t L = a.seqlen;
    CUtensorMap tx, tB, tC, tH, tCB, tz, tout;
    {
        const uint64_t d[4] = {(uint64_t)kP, (uint64_t)a.nheads, L, (uint64_t)a.batch};
        const uint64_t s[3] = {(uint64_t)a.x_stride[2] * 2, (uint64_t)a.x_stride[1] * 2, (uint64_t)a.x_stride[0] * 2};
        const uint32_t bx256[4] = {64, 1, 256, 1}, bx128[4] = {64, 1, 128, 1}, bx64[4] = {64, 1, 64, 1};
        if (!encode_16bit(&tx, fmt, a.x, 4, d, s, stage == 0 ? bx256 : (stage == 2 ? bx128 : bx64)))
            return fail(MB200_ERR_LAUNCH, "ssd: tensor map for x failed");
    }
    {
        const uint64_t d[4] = {(uint64_t)kN, (uint64_t)a.ngroups, L, (uint64_t)a.batch};
        const uint64_t sB[3] = {(uint64_t)a.B_stride[2] * 2, (uint64_t)a.B_stride[1] * 2, (uint64_t)a.B_stride[0] * 2};
        const uint64_t sC[3] = {(uint64_t)a.C_stride[2] * 2, (uint64_t)a.C_stride[1] * 2, (uint64_t)a.C_stride[0] * 2};
        const uint32_t bx256[4] = {64, 1, 256, 1}, bx128[4] = {64, 1, 128, 1};
        if (!encode_16bit(&tB, fmt, a.B, 4, d, sB, stage == 0 ? bx256 : bx128)) return fail(MB200_ERR_LAUNCH, "ssd: tensor map for B failed");
        // only the C.B^T and chunk-scan launches read C (the LOCAL half of a sequence split may not even be given one)
        if (stage == 1 && !encode_16bit(&tC, fmt, a.C, 4, d, sC, bx128)) return fail(MB200_ERR_LAUNCH, "ssd: tensor map for C failed");
    }
    const size_t smem_state = 98304 + 256 + 1024, smem_cb = 98304 + 256 + 1024, smem_scan = kScanSmem;
    if (stage == 2) {
        CUtensorMap tHs;
        const uint64_t d[3] = {(uint64_t)kP, (uint64_t)kN, (uint64_t)a.batch * nc * a.nheads};
        const uint64_t s[2] = {(uint64_t)kP * 2, (uint64_t)kN * kP * 2};
        const uint32_t bx[3] = {64, 128, 1};
        if (!encode_16bit(&tHs, fmt, prev16, 3, d, s, bx)) return fail(MB200_ERR_LAUNCH, "ssd: tensor map for states failed");
        // whole operator: from initial_states, entering states stored.  LOCAL half of a sequence split: from a zero
        // state, entering states stored as they are without the incoming state, plus what the OUTPUT half needs to
        // add that state's share later.
        const bool whole = (a.phases & MB200_SSD_PHASE_OUTPUT) != 0;
        float *aux_prefix = whole ? nullptr : reinterpret_cast<float *>(base + lay.off_aux);
        float *aux_state = whole ? nullptr : reinterpret_cast<float *>(base + lay.off_aux_state);
        float *aux_decay = whole ? nullptr : reinterpret_cast<float *>(base + lay.off_aux_decay);
        const float *init = whole ? a.initial_states : nullptr;
        const int hpg = a.nheads / a.ngroups;
        // Two heads of a group per CTA share the B tile (a fifth less shared-memory and L2 traffic per head), but a
        // CTA then runs 1.6x as long, so only whole waves of such CTAs pay; what is left over runs as pairs if that is
        // more than half a wave and as single heads otherwise.
        const int sms = sm_count(a.device);
        const int64_t pairs = hpg % 2 == 0 ? (int64_t)a.batch * (a.nheads / 2) : 0;
        int64_t paired = pairs / sms * sms;
        if (pairs - paired > sms / 2) paired = pairs;
        if (paired > 0) {
            ensure_dynamic_smem(reinterpret_cast<const void *>(&ssd_tc_state_stream_kernel<T, 2>), (int)StreamCfg<2>::kSmem, a.device);
            ssd_tc_state_stream_kernel<T, 2><<<(unsigned)paired, kStreamThreads, StreamCfg<2>::kSmem, stream>>>(
                tx, tB, tHs, dtb, dAb, init, a.final_states, a.range_decay, aux_prefix, aux_state, aux_decay, 1, nc, a.nheads, hpg, 0, a.seq_idx,
                a.seqlen, status);
            MB200_CHECK_LAUNCH("ssd state stream (tensor core, head pairs)");
        }
        const int64_t singles = (int64_t)a.batch * a.nheads - 2 * paired;
        if (singles > 0) {
            ensure_dynamic_smem(reinterpret_cast<const void *>(&ssd_tc_state_stream_kernel<T, 1>), (int)StreamCfg<1>::kSmem, a.device);
            ssd_tc_state_stream_kernel<T, 1><<<(unsigned)singles, kStreamThreads, StreamCfg<1>::kSmem, stream>>>(
                tx, tB, tHs, dtb, dAb, init, a.final_states, a.range_decay, aux_prefix, aux_state, aux_decay, 1, nc, a.nheads, hpg,
                (int)(2 * paired), a.seq_idx, a.seqlen, status);
        }
        MB200_CHECK_LAUNCH("ssd state stream (tensor core)");
        return MB200_OK;
    }
    if (stage == 0) {
        ensure_dynamic_smem(reinterpret_cast<const void *>(&ssd_tc_chunk_state_kernel<T>), (int)smem_state, a.device);
        ssd_tc_chunk_state_kernel<T><<<dim3(a.nheads, nc, a.batch), kStateThreads, smem_state, stream>>>(tx, tB, dtb, dAb, states, nc, a.nheads,
                                                                                                   a.nheads / a.ngroups, a.seq_idx, a.seqlen, status);
        MB200_CHECK_LAUNCH("ssd chunk_state (tensor core)");
        return MB200_OK;
    }
    if (parts & 1) {
        ensure_dynamic_smem(reinterpret_cast<const void *>(&ssd_tc_cb_kernel<T>), (int)smem_cb, a.device);
        ssd_tc_cb_kernel<T><<<dim3(a.ngroups, nc * 2, a.batch), kThreadsTc, smem_cb, stream>>>(tC, tB, cb16, nc, a.ngroups, status);
        MB200_CHECK_LAUNCH("ssd chunk_cb (tensor core)");
    }
    if (!(parts & 2)) return MB200_OK;       // C.B^T alone (ahead of the exchange of a sequence split): out, z and the states play no part
    if (h_np) {
        const uint64_t d[3] = {(uint64_t)kP, (uint64_t)kN, (uint64_t)a.batch * nc * a.nheads};
        const uint64_t s[2] = {(uint64_t)kP * 2, (uint64_t)kN * kP * 2};
        const uint32_t bx[3] = {64, 64, 1};      // 64 rows n of the [n][p] state: one K half of C.H^T
        if (!encode_16bit(&tH, fmt, prev16, 3, d, s, bx)) return fail(MB200_ERR_LAUNCH, "ssd: tensor map for states failed");
    } else {
        const uint64_t d[3] = {(uint64_t)kN, (uint64_t)kP, (uint64_t)a.batch * nc * a.nheads};
        const uint64_t s[2] = {(uint64_t)kN * 2, (uint64_t)kN * kP * 2};
        const uint32_t bx[3] = {64, 64, 1};
        if (!encode_16bit(&tH, fmt, prev16, 3, d, s, bx)) return fail(MB200_ERR_LAUNCH, "ssd: tensor map for states failed");
    }
    {
        const uint64_t d[3] = {(uint64_t)kQ, (uint64_t)kQ, (uint64_t)a.batch * nc * a.ngroups};
        const uint64_t s[2] = {(uint64_t)kQ * 2, (uint64_t)kQ * kQ * 2};
        const uint32_t bx[3] = {64, 128, 1};
        if (!encode_16bit(&tCB, fmt, cb16, 3, d, s, bx)) return fail(MB200_ERR_LAUNCH, "ssd: tensor map for CB failed");
    }
    {
        const uint64_t d[4] = {(uint64_t)kP, (uint64_t)a.nheads, L, (uint64_t)a.batch};
        const uint32_t bx128[4] = {64, 1, 128, 1};
        const uint64_t so[3] = {(uint64_t)a.out_stride[2] * 2, (uint64_t)a.out_stride[1] * 2, (uint64_t)a.out_stride[0] * 2};
        if (!encode_16bit(&tout, fmt, a.out, 4, d, so, bx128)) return fail(MB200_ERR_LAUNCH, "ssd: tensor map for out failed");
        tz = tout;
        if (a.z) {
            const uint64_t sz[3] = {(uint64_t)a.z_stride[2] * 2, (uint64_t)a.z_stride[1] * 2, (uint64_t)a.z_stride[0] * 2};
            if (!encode_16bit(&tz, fmt, a.z, 4, d, sz, bx128)) return fail(MB200_ERR_LAUNCH, "ssd: tensor map for z failed");
        }
    }
    if (parts & 2) {
        ensure_dynamic_smem(reinterpret_cast<const void *>(&ssd_tc_chunk_scan_kernel<T>), (int)smem_scan, a.device);
        const uint8_t *seq_start = a.seq_idx ? reinterpret_cast<const uint8_t *>(base + lay.off_seq_start) : nullptr;
        const uint8_t *seq_carry = reinterpret_cast<const uint8_t *>(base + lay.off_seq_carry);
        ssd_tc_chunk_scan_kernel<T><<<dim3(a.nheads, nc * 2, a.batch), kScanThreads, smem_scan, stream>>>(tx, tC, tH, tCB, tz, tout, a, dtb, dAb, nc, h_np ? 1 : 0,
                                                                                                          seq_start, seq_carry, status);
        MB200_CHECK_LAUNCH("ssd chunk_scan (tensor core)");
    }
    return MB200_OK;
}

}  // namespace

bool ssd_tc_local_eligible(const mb200_ssd_args &a)
{
    if (a.io_dtype != MB200_BF16 && a.io_dtype != MB200_F16) return false;
    if (a.headdim != kP || a.dstate != kN || a.chunk_size != kQ) return false;
    if (!aligned16(a.x) || !aligned16(a.B) || !mult8(a.x_stride, 3) || !mult8(a.B_stride, 3)) return false;
    if ((int64_t)a.batch * ((a.seqlen + kQ - 1) / kQ) * a.nheads > INT32_MAX) return false;
    return encode_fn() != nullptr;
}

bool ssd_tc_cb_eligible(const mb200_ssd_args &a) { return a.C && aligned16(a.C) && mult8(a.C_stride, 3); }

bool ssd_tc_output_eligible(const mb200_ssd_args &a)
{
    if (!ssd_tc_cb_eligible(a)) return false;
    if (!a.out || !aligned16(a.out) || !mult8(a.out_stride, 3)) return false;
    if (a.z && (!aligned16(a.z) || !mult8(a.z_stride, 3))) return false;
    return true;
}

int ssd_tc_chunk_state(const mb200_ssd_args &a, const SsdScratch &lay, cudaStream_t stream)
{
    return a.io_dtype == MB200_BF16 ? run_tc<__nv_bfloat16>(a, lay, 0, false, stream) : run_tc<__half>(a, lay, 0, false, stream);
}

int ssd_tc_cb_and_scan(const mb200_ssd_args &a, const SsdScratch &lay, bool states_np, cudaStream_t stream, int parts)
{
    return a.io_dtype == MB200_BF16 ? run_tc<__nv_bfloat16>(a, lay, 1, states_np, stream, parts)
                                    : run_tc<__half>(a, lay, 1, states_np, stream, parts);
}

// One (batch, head) per CTA: worth it once those fill at least half of the SMs.
bool ssd_tc_stream_eligible(const mb200_ssd_args &a)
{
    return (int64_t)a.batch * a.nheads >= kStreamMinUnits;
}

template <typename T>
int run_incoming(const mb200_ssd_args &a, const SsdScratch &lay, cudaStream_t stream)
{
    char *base = static_cast<char *>(a.scratch);
    const float *aux_state = reinterpret_cast<const float *>(base + lay.off_aux_state);
    const float *aux_decay = reinterpret_cast<const float *>(base + lay.off_aux_decay);
    const int64_t PN = (int64_t)kP * kN;
    if (!a.initial_states) {       // nothing came in: the entering states stand, the end state is the local one
        if (a.final_states) {
            const cudaError_t e = cudaMemcpyAsync(a.final_states, aux_state, sizeof(float) * (size_t)a.batch * a.nheads * PN,
                                                  cudaMemcpyDeviceToDevice, stream);
            if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "ssd: copying the range state: %s", cudaGetErrorString(e));
        }
        return MB200_OK;
    }
    ssd_incoming_state_kernel<T><<<dim3((lay.nchunks + kFixChunks - 1) / kFixChunks, a.nheads, a.batch), 256, 0, stream>>>(
        reinterpret_cast<T *>(base + lay.off_prev16), a.initial_states, reinterpret_cast<const float *>(base + lay.off_aux), aux_state,
        aux_decay, a.final_states, lay.nchunks, a.nheads);
    MB200_CHECK_LAUNCH("ssd incoming state");
    return MB200_OK;
}

int ssd_tc_apply_incoming(const mb200_ssd_args &a, const SsdScratch &lay, cudaStream_t stream)
{
    return a.io_dtype == MB200_BF16 ? run_incoming<__nv_bfloat16>(a, lay, stream) : run_incoming<__half>(a, lay, stream);
}

int ssd_tc_state_stream(const mb200_ssd_args &a, const SsdScratch &lay, cudaStream_t stream)
{
    return a.io_dtype == MB200_BF16 ? run_tc<__nv_bfloat16>(a, lay, 2, true, stream) : run_tc<__half>(a, lay, 2, true, stream);
}

}  // namespace mb200

