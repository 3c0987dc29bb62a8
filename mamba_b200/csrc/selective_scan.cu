// Mamba-1 selective scan forward for sm_100a.
//
// Work split: a CTA owns kWarps*cpw consecutive channels of one (batch, group) and walks the
// sequence in tiles of kTile = 32 lanes x kItems steps.  For every tile the B and C rows of the
// group (dstate x kTile, shared by all channels of the CTA) are staged once in shared memory as
// fp32 in a packet-swizzled layout; a warp then takes one channel at a time: each lane loads its
// kItems consecutive steps of u, delta (16-byte packets), and for each state n
//   1. forms a_i = 2^(dt_i A_n log2e), b_i = dt_i u_i B_{n,i}                (registers)
//   2. folds them sequentially into the lane aggregate (prod a, h_local)      (prod a = 2^(A sum dt))
//   3. runs a 5-step shuffle scan over the lanes with (a1,b1)o(a0,b0) = (a1 a0, a1 b0 + b1)
//   4. re-runs the recurrence from the true incoming state and accumulates y_i += C_{n,i} h_i
// The state carried between tiles lives in shared memory (one float per channel and state), so any
// dstate <= 256 works; states are processed in blocks of kStateBlock with B/C re-staged per block.
// Steps past seqlen get dt = 0, u = 0, i.e. the identity (1, 0), so the final state is exact.
#include <type_traits>

#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kItems = 16;
constexpr int kTile = 32 * kItems;        // 512 steps
constexpr int kStateBlock = 16;
constexpr int kPackets = kTile / 4;       // float4 packets per staged row

// Packet q of a staged row is stored at q ^ ((q >> 2) & 7): the four packets a lane reads back to
// back (4*lane + j) then fall in distinct bank groups across each quarter warp.
__device__ __forceinline__ int swz(int q) { return q ^ ((q >> 2) & 7); }

template <typename T>
__device__ __forceinline__ void load_items(const T *row, int t0, int L, bool vec_ok, float (&v)[kItems])
{
    constexpr int VEC = 16 / sizeof(T);
    if (vec_ok && t0 + kItems <= L) {
#pragma unroll
        for (int k = 0; k < kItems / VEC; ++k) {
            Vec16<T> p;
            p.load(row + t0 + k * VEC);
            float f[VEC];
            p.unpack(f);
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[k * VEC + i] = f[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i < kItems; ++i) v[i] = (t0 + i < L) ? to_float(row[t0 + i]) : 0.f;
    }
}

template <typename T>
__device__ __forceinline__ void store_items(T *row, int t0, int L, bool vec_ok, const float (&v)[kItems])
{
    constexpr int VEC = 16 / sizeof(T);
    if (vec_ok && t0 + kItems <= L) {
#pragma unroll
        for (int k = 0; k < kItems / VEC; ++k) {
            float f[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) f[i] = v[k * VEC + i];
            Vec16<T> p;
            p.pack(f);
            p.store(row + t0 + k * VEC);
        }
    } else {
#pragma unroll
        for (int i = 0; i < kItems; ++i)
            if (t0 + i < L) row[t0 + i] = from_float<T>(v[i]);
    }
}

// Stage rows [n0, n0+kStateBlock) x steps [tile0, tile0+kTile) of a variable B or C as fp32.
template <typename T>
__device__ __forceinline__ void stage_rows(float *dst, const T *src, int64_t n_stride, int n0, int N, int tile0, int L,
                                           bool vec_ok)
{
    for (int idx = threadIdx.x; idx < kStateBlock * kPackets; idx += kThreads) {
        const int n = idx / kPackets, q = idx % kPackets;
        const int t = tile0 + q * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n0 + n < N) {
            const T *p = src + (int64_t)(n0 + n) * n_stride + t;
            if (vec_ok && t + 4 <= L) {
                if constexpr (sizeof(T) == 4) {
                    v = *reinterpret_cast<const float4 *>(p);
                } else {
                    const uint2 raw = *reinterpret_cast<const uint2 *>(p);
                    const T *e = reinterpret_cast<const T *>(&raw);
                    v = make_float4(to_float(e[0]), to_float(e[1]), to_float(e[2]), to_float(e[3]));
                }
            } else {
                if (t + 0 < L) v.x = to_float(p[0]);
                if (t + 1 < L) v.y = to_float(p[1]);
                if (t + 2 < L) v.z = to_float(p[2]);
                if (t + 3 < L) v.w = to_float(p[3]);
            }
        }
        reinterpret_cast<float4 *>(dst)[n * kPackets + swz(q)] = v;
    }
}

// Pulls the 16-byte packets a lane will need for steps [t0, t0+kItems) of `row` into L1 ahead of use.
template <typename T>
__device__ __forceinline__ void prefetch_items(const T *row, int t0, int L)
{
    if (t0 < L) {
        const char *p = reinterpret_cast<const char *>(row + t0);
#pragma unroll
        for (int o = 0; o < (int)(kItems * sizeof(T)); o += 32) asm volatile("prefetch.global.L1 [%0];" ::"l"(p + o));
    }
}

__device__ __forceinline__ void read_items(const float *rowbase, int lane, float (&v)[kItems])
{
    const float4 *r = reinterpret_cast<const float4 *>(rowbase);
#pragma unroll
    for (int j = 0; j < kItems / 4; ++j) {
        const float4 p = r[swz(lane * (kItems / 4) + j)];
        v[4 * j + 0] = p.x; v[4 * j + 1] = p.y; v[4 * j + 2] = p.z; v[4 * j + 3] = p.w;
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
scan_fwd_kernel(const mb200_scan_args a, const int cpw, const int nblocks, const int npad, const int vec_flags)
{
    extern __shared__ __align__(16) float smem[];
    float *Bs = smem;                                // kStateBlock x kTile
    float *Cs = Bs + kStateBlock * kTile;            // kStateBlock x kTile
    float *A2s = Cs + kStateBlock * kTile;           // channels x npad : A log2e
    float *run = A2s + kWarps * cpw * npad;          // channels x npad : state entering the tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.y;
    const int N = a.dstate, L = a.seqlen;
    const int per_group = a.dim / a.ngroups;
    const int chans = kWarps * cpw;
    const int tiles_per_group = (per_group + chans - 1) / chans;
    const int g = blockIdx.x / tiles_per_group;
    const int d_first = g * per_group + (blockIdx.x % tiles_per_group) * chans;
    const int d_end = (g + 1) * per_group;
    const bool io_vec = vec_flags & 1, bc_vec = vec_flags & 2;

    for (int i = threadIdx.x; i < chans * npad; i += kThreads) {
        const int cl = i / npad, n = i % npad;
        const int d = d_first + cl;
        A2s[i] = (d < d_end && n < N) ? a.A[(int64_t)d * a.A_stride[0] + (int64_t)n * a.A_stride[1]] * kLog2e : 0.f;
        run[i] = 0.f;
    }

    const T *Bg = a.B_variable ? static_cast<const T *>(a.B) + (int64_t)b * a.B_stride[0] + (int64_t)g * a.B_stride[1] : nullptr;
    const T *Cg = a.C_variable ? static_cast<const T *>(a.C) + (int64_t)b * a.C_stride[0] + (int64_t)g * a.C_stride[1] : nullptr;

    const int ntiles = (L + kTile - 1) / kTile;
    for (int tile = 0; tile < ntiles; ++tile) {
        const int tile0 = tile * kTile;
        const int t0 = tile0 + lane * kItems;
        for (int c = 0; c < cpw; ++c) {
            const int cl = warp * cpw + c;
            const int d = d_first + cl;
            const bool live = d < d_end;
            float dl[kItems], du[kItems], y[kItems];
            float sum_dt = 0.f;
            if (live) {
                const T *urow = static_cast<const T *>(a.u) + (int64_t)b * a.u_stride[0] + (int64_t)d * a.u_stride[1];
                const T *drow = static_cast<const T *>(a.delta) + (int64_t)b * a.delta_stride[0] + (int64_t)d * a.delta_stride[1];
                float uu[kItems];
                load_items(urow, t0, L, io_vec, uu);
                load_items(drow, t0, L, io_vec, dl);
                const float bias = a.delta_bias ? a.delta_bias[d] : 0.f;
                const float Dd = a.D ? a.D[d] : 0.f;
#pragma unroll
                for (int i = 0; i < kItems; ++i) {
                    float v = dl[i] + bias;
                    if (a.delta_softplus) v = fast_softplus20(v);
                    if (t0 + i >= L) v = 0.f;
                    dl[i] = v;
                    sum_dt += v;
                    du[i] = v * uu[i];
                    y[i] = Dd * uu[i];
                }
                // while this channel's states are scanned, fetch what comes next: its own z row and
                // the u / delta rows of the warp's next (channel, tile)
                if (a.z) prefetch_items(static_cast<const T *>(a.z) + (int64_t)b * a.z_stride[0] + (int64_t)d * a.z_stride[1], t0, L);
                const int dn = (c + 1 < cpw) ? d + 1 : d_first + warp * cpw;
                const int tn = (c + 1 < cpw) ? t0 : t0 + kTile;
                if (dn < d_end) {
                    prefetch_items(static_cast<const T *>(a.u) + (int64_t)b * a.u_stride[0] + (int64_t)dn * a.u_stride[1], tn, L);
                    prefetch_items(static_cast<const T *>(a.delta) + (int64_t)b * a.delta_stride[0] + (int64_t)dn * a.delta_stride[1], tn, L);
                }
            }
            for (int nb = 0; nb < nblocks; ++nb) {
                const int n0 = nb * kStateBlock;
                if (c == 0 || nblocks > 1) {
                    __syncthreads();   // the previous contents of Bs/Cs are no longer being read
                    if (a.B_variable) stage_rows(Bs, Bg, a.B_stride[2], n0, N, tile0, L, bc_vec);
                    if (a.C_variable) stage_rows(Cs, Cg, a.C_stride[2], n0, N, tile0, L, bc_vec);
                    __syncthreads();
                }
                if (!live) continue;
                const int ns = min(kStateBlock, N - n0);
                for (int s = 0; s < ns; ++s) {
                    const int n = n0 + s;
                    const float A2 = A2s[cl * npad + n];
                    float av[kItems], bv[kItems], tmp[kItems];
                    if (a.B_variable) {
                        read_items(Bs + s * kTile, lane, tmp);
                    } else {
                        const float Bc = static_cast<const float *>(a.B)[(int64_t)d * a.B_stride[0] + (int64_t)n * a.B_stride[1]];
#pragma unroll
                        for (int i = 0; i < kItems; ++i) tmp[i] = Bc;
                    }
                    float h = 0.f;
#pragma unroll
                    for (int i = 0; i < kItems; ++i) {
                        av[i] = ex2(dl[i] * A2);
                        bv[i] = du[i] * tmp[i];
                        h = fmaf(av[i], h, bv[i]);
                    }
                    // lane aggregate, then inclusive scan over lanes
                    float P = ex2(sum_dt * A2), H = h;
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const float Pp = __shfl_up_sync(0xffffffffu, P, o);
                        const float Hp = __shfl_up_sync(0xffffffffu, H, o);
                        if (lane >= o) {
                            H = fmaf(P, Hp, H);
                            P *= Pp;
                        }
                    }
                    float Pe = __shfl_up_sync(0xffffffffu, P, 1);
                    float He = __shfl_up_sync(0xffffffffu, H, 1);
                    if (lane == 0) { Pe = 1.f; He = 0.f; }
                    const float h_run = run[cl * npad + n];
                    h = fmaf(Pe, h_run, He);                   // state entering this lane's steps
                    if (a.C_variable) {
                        read_items(Cs + s * kTile, lane, tmp);
                    } else {
                        const float Cc = static_cast<const float *>(a.C)[(int64_t)d * a.C_stride[0] + (int64_t)n * a.C_stride[1]];
#pragma unroll
                        for (int i = 0; i < kItems; ++i) tmp[i] = Cc;
                    }
#pragma unroll
                    for (int i = 0; i < kItems; ++i) {
                        h = fmaf(av[i], h, bv[i]);
                        y[i] = fmaf(h, tmp[i], y[i]);
                    }
                    if (lane == 31) run[cl * npad + n] = h;    // read back only by this warp, next tile
                }
                __syncwarp();
            }
            if (live) {
                T *orow = static_cast<T *>(a.out) + (int64_t)b * a.out_stride[0] + (int64_t)d * a.out_stride[1];
                if (a.z) {
                    if (a.out_pregate) {
                        T *prow = static_cast<T *>(a.out_pregate) + (int64_t)b * a.pregate_stride[0] + (int64_t)d * a.pregate_stride[1];
                        store_items(prow, t0, L, io_vec, y);
                    }
                    const T *zrow = static_cast<const T *>(a.z) + (int64_t)b * a.z_stride[0] + (int64_t)d * a.z_stride[1];
                    float zz[kItems];
                    load_items(zrow, t0, L, io_vec, zz);
#pragma unroll
                    for (int i = 0; i < kItems; ++i) y[i] *= fast_silu(zz[i]);
                }
                store_items(orow, t0, L, io_vec, y);
            }
        }
    }
    if (a.last_state) {
        __syncwarp();
        for (int c = 0; c < cpw; ++c) {
            const int cl = warp * cpw + c;
            const int d = d_first + cl;
            if (d >= d_end) continue;
            for (int n = lane; n < N; n += 32)
                a.last_state[((int64_t)b * a.dim + d) * N + n] = run[cl * npad + n];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Channel-parallel variant for dstate <= 16 with input-dependent B and C: time is sequential, a
// channel belongs to a PAIR of lanes that split its states between them (16 channels per warp).
// All lanes of a warp are at the same step, so B_t and C_t are warp-uniform (broadcast reads of a
// tiny per-warp shared tile) and the only loop-carried dependence is one FMA per state: no scan tree,
// no re-evaluation -- 4 FMA-pipe + 1 MUFU instruction per (step, state).  The pair also splits the
// per-step scalar work: each lane evaluates softplus(dt) and silu(z) for half of the block's steps
// and the partner gets dt by shuffle; the two partial outputs meet in one more shuffle.  A lane
// streams its channel's rows 32 bytes at a time (whole sectors) with the next block prefetched into
// L1; warps never synchronise with each other, so a CTA is one warp and the grid spreads evenly.
constexpr int kSeqBytes = 32;   // bytes of one row a lane moves per block (two 16-byte packets)
#ifndef MB200_SEQ_AHEAD
#define MB200_SEQ_AHEAD 2
#endif
constexpr int kSeqAhead = MB200_SEQ_AHEAD;   // how many blocks ahead the L1 prefetch runs
#ifndef MB200_SEQ_DT_UPFRONT
#define MB200_SEQ_DT_UPFRONT 0
#endif
// Register cap: 2560 one-warp CTAs of the 2.8B-layer shape must all be resident at once (17.3 per SM);
// 96 registers allow 20 per SM, 104 or more leave a second, nearly empty wave (0.70 ms -> 0.93 ms measured).
#ifndef MB200_SEQ_MAXNREG
#define MB200_SEQ_MAXNREG 96
#endif

template <typename T> struct SeqRaw { uint4 v[2]; };

template <typename T>
__device__ __forceinline__ float seq_get(const SeqRaw<T> &r, int i)
{
    const uint32_t *w = reinterpret_cast<const uint32_t *>(r.v);
    if constexpr (sizeof(T) == 4) {
        return __uint_as_float(w[i]);
    } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        const uint32_t x = w[i >> 1];
        return __uint_as_float((i & 1) ? (x & 0xffff0000u) : (x << 16));
    } else {
        const uint32_t x = w[i >> 1];
        return __half2float(__ushort_as_half((unsigned short)((i & 1) ? (x >> 16) : (x & 0xffffu))));
    }
}

template <typename T>
__device__ __forceinline__ SeqRaw<T> seq_load(const T *row, int t0, int L, bool vec_ok)
{
    constexpr int TB = kSeqBytes / sizeof(T);
    SeqRaw<T> r;
    if (vec_ok && t0 + TB <= L) {
        r.v[0] = *reinterpret_cast<const uint4 *>(row + t0);
        r.v[1] = *(reinterpret_cast<const uint4 *>(row + t0) + 1);
    } else {
        T *e = reinterpret_cast<T *>(r.v);
#pragma unroll
        for (int i = 0; i < TB; ++i) e[i] = (t0 + i < L) ? row[t0 + i] : from_float<T>(0.f);
    }
    return r;
}

template <typename T>
__device__ __forceinline__ void seq_prefetch(const T *row, int t0, int L)
{
    if (t0 < L) asm volatile("prefetch.global.L1 [%0];" ::"l"(row + t0));
}

template <typename T, int NS>
__global__ void __maxnreg__(MB200_SEQ_MAXNREG) scan_seq_kernel(const mb200_scan_args a, const int vec_flags)
{
    constexpr int TB = kSeqBytes / sizeof(T);          // steps per block: 16 (16-bit) or 8 (fp32)
    constexpr int HS = NS / 2;                         // states per lane
    constexpr int HP = TB / 2;                         // steps per 16-byte packet
    __shared__ __align__(16) float Bs[TB * NS], Cs[TB * NS];
    const int lane = threadIdx.x;
    const int half = lane & 1;                         // which half of the states / of the block's steps is mine
    const int N = a.dstate, L = a.seqlen;
    const int per_group = a.dim / a.ngroups;
    const int blocks_per_group = (per_group + 15) / 16;
    const int b = blockIdx.y;
    const int g = blockIdx.x / blocks_per_group;
    const int d = g * per_group + (blockIdx.x % blocks_per_group) * 16 + (lane >> 1);
    const bool live = d < (g + 1) * per_group;
    const int dc = live ? d : g * per_group;            // idle lanes shadow a valid channel, store nothing
    const bool io_vec = vec_flags & 1, bc_vec = vec_flags & 2;

    // states live as packed fp32 pairs: every multiply / FMA of the recurrence is one f32x2 instruction
    uint64_t A2[HS / 2], h[HS / 2];
#pragma unroll
    for (int j = 0; j < HS / 2; ++j) {
        float av[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int n = half * HS + 2 * j + e;
            av[e] = n < N ? a.A[(int64_t)dc * a.A_stride[0] + (int64_t)n * a.A_stride[1]] * kLog2e : 0.f;
        }
        A2[j] = pack2(av[0], av[1]);
        h[j] = pack2(0.f, 0.f);
    }
    const float bias = a.delta_bias ? a.delta_bias[dc] : 0.f;
    const float Dd = (a.D && half == 0) ? a.D[dc] : 0.f;   // the skip term is added once per pair
    const T *urow = static_cast<const T *>(a.u) + (int64_t)b * a.u_stride[0] + (int64_t)dc * a.u_stride[1];
    const T *drow = static_cast<const T *>(a.delta) + (int64_t)b * a.delta_stride[0] + (int64_t)dc * a.delta_stride[1];
    const T *zrow = a.z ? static_cast<const T *>(a.z) + (int64_t)b * a.z_stride[0] + (int64_t)dc * a.z_stride[1] : nullptr;
    T *orow = static_cast<T *>(a.out) + (int64_t)b * a.out_stride[0] + (int64_t)dc * a.out_stride[1];
    T *prow = (a.z && a.out_pregate) ? static_cast<T *>(a.out_pregate) + (int64_t)b * a.pregate_stride[0] + (int64_t)dc * a.pregate_stride[1] : nullptr;

    // B/C staging: the block's tile is N rows x 32 bytes = N x 2 packets; lane -> (row lane/2, packet lane%2)
    const int sn = lane >> 1;
    const T *Bsrc = static_cast<const T *>(a.B) + (int64_t)b * a.B_stride[0] + (int64_t)g * a.B_stride[1] + (int64_t)sn * a.B_stride[2];
    const T *Csrc = static_cast<const T *>(a.C) + (int64_t)b * a.C_stride[0] + (int64_t)g * a.C_stride[1] + (int64_t)sn * a.C_stride[2];
    auto bc_stage = [&](float *dst, const T *src, int t0) {
        if (sn < NS) {
            uint4 r = make_uint4(0, 0, 0, 0);
            const int ts = t0 + half * HP;
            if (sn < N) {
                if (bc_vec && ts + HP <= L) {
                    r = *reinterpret_cast<const uint4 *>(src + ts);
                } else {
                    T *e = reinterpret_cast<T *>(&r);
#pragma unroll
                    for (int i = 0; i < HP; ++i) e[i] = (ts + i < L) ? src[ts + i] : from_float<T>(0.f);
                }
            }
            const T *e = reinterpret_cast<const T *>(&r);
#pragma unroll
            for (int i = 0; i < HP; ++i) dst[(half * HP + i) * NS + sn] = to_float(e[i]);
        }
    };

    const int nblk = (L + TB - 1) / TB;
    for (int blk = 0; blk < nblk; ++blk) {
        const int t0 = blk * TB;
        bc_stage(Bs, Bsrc, t0);
        bc_stage(Cs, Csrc, t0);
        const SeqRaw<T> ru = seq_load(urow, t0, L, io_vec), rd = seq_load(drow, t0, L, io_vec);
        SeqRaw<T> rz;
        if (zrow) rz = seq_load(zrow, t0, L, io_vec);
        {   // sectors of a later block start moving while this block is computed (kSeqAhead blocks of lead)
            const int tp = t0 + kSeqAhead * TB;
            seq_prefetch(urow, tp, L);
            seq_prefetch(drow, tp, L);
            if (zrow) seq_prefetch(zrow, tp, L);
            if (sn < N) {
                seq_prefetch(Bsrc, tp + half * HP, L);
                seq_prefetch(Csrc, tp + half * HP, L);
            }
        }
        // my half of the block's dt values; the partner's arrive by shuffle inside the step loop
        float dtm[HP];
#pragma unroll
        for (int i = 0; i < HP; ++i) {
            float v = (half ? seq_get<T>(rd, HP + i) : seq_get<T>(rd, i)) + bias;   // compile-time register indices
            if (a.delta_softplus) v = fast_softplus20(v);
            if (t0 + half * HP + i >= L) v = 0.f;
            dtm[i] = v;
        }
        __syncwarp();               // B/C tile of this block is in place
#if MB200_SEQ_DT_UPFRONT
        // the partner's half of the dt values, exchanged once per block so that no shuffle sits at the head of a
        // step's dependency chain
        float dta[TB];
#pragma unroll
        for (int i = 0; i < HP; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, dtm[i], 1);
            dta[i] = half ? other : dtm[i];
            dta[HP + i] = half ? dtm[i] : other;
        }
#endif
        float ym[HP];               // outputs of my half of the steps
#pragma unroll
        for (int i = 0; i < TB; ++i) {
            const float uu = seq_get<T>(ru, i);
#if MB200_SEQ_DT_UPFRONT
            const float dl = dta[i];
#else
            const float dl = __shfl_sync(0xffffffffu, dtm[i % HP], (lane & ~1) | (i / HP));
#endif
            const float du = dl * uu;
            const uint64_t dl2 = pack2(dl, dl), du2 = pack2(du, du);
            uint64_t ya = pack2(Dd * uu, 0.f), yb = pack2(0.f, 0.f);
            const ulonglong2 *Bt = reinterpret_cast<const ulonglong2 *>(Bs + i * NS + half * HS);
            const ulonglong2 *Ct = reinterpret_cast<const ulonglong2 *>(Cs + i * NS + half * HS);
#pragma unroll
            for (int q = 0; q < HS / 4; ++q) {
                const ulonglong2 bb = Bt[q], cc = Ct[q];
                float x0, x1;
                unpack2(mul2(dl2, A2[2 * q]), x0, x1);
                h[2 * q] = fma2(pack2(ex2(x0), ex2(x1)), h[2 * q], mul2(du2, bb.x));
                ya = fma2(h[2 * q], cc.x, ya);
                unpack2(mul2(dl2, A2[2 * q + 1]), x0, x1);
                h[2 * q + 1] = fma2(pack2(ex2(x0), ex2(x1)), h[2 * q + 1], mul2(du2, bb.y));
                yb = fma2(h[2 * q + 1], cc.y, yb);
            }
            float s0, s1, s2, s3;
            unpack2(ya, s0, s1);
            unpack2(yb, s2, s3);
            const float y = (s0 + s1) + (s2 + s3);
            const float yt = y + __shfl_xor_sync(0xffffffffu, y, 1);
            if ((i / HP) == 0) { if (!half) ym[i % HP] = yt; } else { if (half) ym[i % HP] = yt; }
        }
        __syncwarp();               // every lane is done with the B/C tile before the next block overwrites it
        if (live) {
            const int ts = t0 + half * HP;
            float yg[HP];
#pragma unroll
            for (int i = 0; i < HP; ++i) {
                float zz = 0.f;
                if (zrow) zz = half ? seq_get<T>(rz, HP + i) : seq_get<T>(rz, i);
                yg[i] = zrow ? ym[i] * fast_silu(zz) : ym[i];
            }
            auto put = [&](T *row, const float (&v)[HP]) {
                if (io_vec && ts + HP <= L) {
                    uint4 o;
                    T *e = reinterpret_cast<T *>(&o);
#pragma unroll
                    for (int i = 0; i < HP; ++i) e[i] = from_float<T>(v[i]);
                    *reinterpret_cast<uint4 *>(row + ts) = o;
                } else {
#pragma unroll
                    for (int i = 0; i < HP; ++i)
                        if (ts + i < L) row[ts + i] = from_float<T>(v[i]);
                }
            };
            put(orow, yg);
            if (prow) put(prow, ym);
        }
    }
    if (a.last_state && live) {
        float *ls = a.last_state + ((int64_t)b * a.dim + d) * N;
#pragma unroll
        for (int j = 0; j < HS / 2; ++j) {
            float lo, hi;
            unpack2(h[j], lo, hi);
            if (half * HS + 2 * j < N) ls[half * HS + 2 * j] = lo;
            if (half * HS + 2 * j + 1 < N) ls[half * HS + 2 * j + 1] = hi;
        }
    }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
int launch_scan(const mb200_scan_args &a, cudaStream_t stream)
{
    constexpr int VEC = 16 / sizeof(T);
    const int N = a.dstate;
    const int nblocks = (N + kStateBlock - 1) / kStateBlock;
    const int per_group = a.dim / a.ngroups;
    // more channels per staged B/C tile when the states fit one block and there is enough work
    int cpw = 1;
    if (nblocks == 1 && per_group >= 2 * kWarps && (int64_t)a.batch * a.dim >= 8 * kWarps * 2 * 148) cpw = 2;
    const int chans = kWarps * cpw;
    const int npad = N;
    auto strides_ok = [&](const int64_t *s) { return s[0] % VEC == 0 && s[1] % VEC == 0; };
    bool io_vec = aligned16(a.u) && aligned16(a.delta) && aligned16(a.out) && strides_ok(a.u_stride) &&
                  strides_ok(a.delta_stride) && strides_ok(a.out_stride);
    if (a.z) io_vec = io_vec && aligned16(a.z) && strides_ok(a.z_stride);
    if (a.z && a.out_pregate) io_vec = io_vec && aligned16(a.out_pregate) && strides_ok(a.pregate_stride);
    // staging reads 4 elements at a time: 8 bytes for 16-bit types, 16 for fp32
    const int bc_align = sizeof(T) == 4 ? 16 : 8;
    bool bc_vec = true;
    if (a.B_variable)
        bc_vec = bc_vec && (reinterpret_cast<uintptr_t>(a.B) % bc_align == 0) && a.B_stride[0] % 4 == 0 &&
                 a.B_stride[1] % 4 == 0 && a.B_stride[2] % 4 == 0;
    if (a.C_variable)
        bc_vec = bc_vec && (reinterpret_cast<uintptr_t>(a.C) % bc_align == 0) && a.C_stride[0] % 4 == 0 &&
                 a.C_stride[1] % 4 == 0 && a.C_stride[2] % 4 == 0;
    const int vec_flags = (io_vec ? 1 : 0) | (bc_vec ? 2 : 0);
    // Enough independent channels to give every SM a few warps: one lane per channel, time sequential.
    if (N <= 16 && a.B_variable && a.C_variable && (int64_t)a.batch * a.dim >= 2LL * 32 * 148) {
        // the B/C tile is fetched in 16-byte packets here
        const bool bc16 = bc_vec && aligned16(a.B) && aligned16(a.C) && a.B_stride[0] % VEC == 0 && a.B_stride[1] % VEC == 0 &&
                          a.B_stride[2] % VEC == 0 && a.C_stride[0] % VEC == 0 && a.C_stride[1] % VEC == 0 && a.C_stride[2] % VEC == 0;
        const int flags = (io_vec ? 1 : 0) | (bc16 ? 2 : 0);
        dim3 grid(a.ngroups * ((per_group + 15) / 16), a.batch);
        if (N <= 8) scan_seq_kernel<T, 8><<<grid, 32, 0, stream>>>(a, flags);
        else scan_seq_kernel<T, 16><<<grid, 32, 0, stream>>>(a, flags);
        return MB200_OK;
    }
    const size_t smem = sizeof(float) * (2 * kStateBlock * kTile + 2 * (size_t)chans * npad);
    static_assert(2 * kStateBlock * kTile * sizeof(float) + 2 * kWarps * 2 * 256 * sizeof(float) <= 227 * 1024, "smem budget");
    cudaError_t e = cudaFuncSetAttribute(scan_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "selective_scan: shared memory opt-in (%zu B): %s", smem, cudaGetErrorString(e));
    const int tiles_per_group = (per_group + chans - 1) / chans;
    dim3 grid(a.ngroups * tiles_per_group, a.batch);
    scan_fwd_kernel<T><<<grid, kThreads, smem, stream>>>(a, cpw, nblocks, npad, vec_flags);
    return MB200_OK;
}

}  // namespace
}  // namespace mb200

extern "C" int mb200_selective_scan_fwd(const mb200_scan_args *args, void *stream_)
{
    using namespace mb200;
    if (!args) return fail(MB200_ERR_BAD_ARG, "selective_scan_fwd: args is NULL");
    const mb200_scan_args &a = *args;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MB200_CHECK_ARG(a.batch >= 0 && a.dim > 0 && a.seqlen >= 0 && a.dstate > 0 && a.ngroups > 0,
                    "selective_scan_fwd: bad sizes (batch %d dim %d seqlen %d dstate %d ngroups %d)", a.batch, a.dim,
                    a.seqlen, a.dstate, a.ngroups);
    MB200_CHECK_ARG(a.dstate <= 256, "selective_scan only supports state dimension <= 256");
    MB200_CHECK_ARG(a.dim % a.ngroups == 0, "selective_scan_fwd: dim must be divisible by ngroups");
    MB200_CHECK_ARG(a.io_dtype == MB200_F32 || a.io_dtype == MB200_F16 || a.io_dtype == MB200_BF16,
                    "selective_scan_fwd: unknown io_dtype %d", a.io_dtype);
    MB200_CHECK_ARG(a.batch <= 65535, "selective_scan_fwd: batch must be <= 65535");
    MB200_CHECK_ARG(!a.out_pregate || a.z, "selective_scan_fwd: out_pregate is only meaningful with z");
    if (a.batch == 0) return MB200_OK;   // nothing to do; empty tensors carry NULL pointers
    MB200_CHECK_ARG(a.u && a.delta && a.A && a.B && a.C && a.out, "selective_scan_fwd: a required tensor is NULL");
    if (int rc = enter_device(a.device)) return rc;
    if (a.seqlen == 0) {
        if (a.last_state) {
            cudaError_t e = cudaMemsetAsync(a.last_state, 0, sizeof(float) * (size_t)a.batch * a.dim * a.dstate, stream);
            if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "selective_scan_fwd: memset: %s", cudaGetErrorString(e));
        }
        return MB200_OK;
    }
    int rc;
    if (a.io_dtype == MB200_F32) rc = launch_scan<float>(a, stream);
    else if (a.io_dtype == MB200_BF16) rc = launch_scan<__nv_bfloat16>(a, stream);
    else rc = launch_scan<__half>(a, stream);
    if (rc) return rc;
    MB200_CHECK_LAUNCH("selective_scan_fwd");
    return MB200_OK;
}
