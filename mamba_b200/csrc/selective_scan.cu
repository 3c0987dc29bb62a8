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
#include "tc_sm100.cuh"
#include "tensor_map.cuh"

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
// channel belongs to FOUR lanes that split its states between them (8 channels per warp).  All
// lanes of a warp are at the same step, so B_t and C_t are warp-uniform (broadcast reads of a small
// shared tile) and the only loop-carried dependence is one FMA per state: no scan tree, no
// re-evaluation -- 4 FMA-pipe + 1 MUFU instruction per (step, state).  Four states per lane keep a
// lane at 56 registers, so 36 warps are resident per SM and the MUFU, FMA and load latencies of one
// warp hide behind the others (with two lanes per channel and 96 registers the same loop ran at 17
// warps per SM and was 2-3 % slower; one lane per channel needed 207 registers and a second wave).
// A lane owns a quarter of each block's steps for the per-step scalars (softplus(dt), silu(z), the
// output store: 8 bytes of each row per block); dt reaches the other three lanes by shuffle and the
// four partial outputs meet in two butterfly shuffles.  A lane streams its channel's u row 32 bytes
// at a time (whole sectors) with later blocks prefetched into L1.  The warps of a CTA share one
// double-buffered B/C tile: the staging threads fetch the next block's packets into registers before
// the block's steps and write them to the other buffer afterwards, so one CTA barrier per block
// suffices.
constexpr int kSeqBytes = 32;   // bytes of one u row a lane moves per block (two 16-byte packets)
constexpr int kSeqAhead = 2;    // how many blocks ahead the L1 prefetch runs
constexpr int kQuadWarps = 4;   // warps per CTA of the four-lanes-per-channel kernel
// CTAs per SM the register allocation must allow: the 1280 four-warp CTAs of the 2.8B-layer shape must
// all be resident at once (8.65 per SM); 9 per SM means 56 registers per lane.  With 64 registers only 8
// fit, the last 96 CTAs form a second wave and the step takes 0.84 ms instead of 0.69 ms.
constexpr int kQuadMinBlocks = 9;

template <typename T>
__device__ __forceinline__ void seq_prefetch(const T *row, int t0, int L)
{
    if (t0 < L) asm volatile("prefetch.global.L1 [%0];" ::"l"(row + t0));
}

template <typename T>
__device__ __forceinline__ float words_get(const uint32_t *w, int i)
{
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

// NB bytes (8, 16 or 32) of a row starting at element t0, zero-filled past L
template <typename T, int NB>
__device__ __forceinline__ void row_load(uint32_t (&w)[NB / 4], const T *row, int t0, int L, bool vec_ok)
{
    constexpr int NE = NB / sizeof(T);
    if (vec_ok && t0 + NE <= L) {
        if constexpr (NB == 8) {
            const uint2 r = *reinterpret_cast<const uint2 *>(row + t0);
            w[0] = r.x; w[1] = r.y;
        } else {
#pragma unroll
            for (int k = 0; k < NB / 16; ++k) {
                const uint4 r = *(reinterpret_cast<const uint4 *>(row + t0) + k);
                w[4 * k] = r.x; w[4 * k + 1] = r.y; w[4 * k + 2] = r.z; w[4 * k + 3] = r.w;
            }
        }
    } else {
        T *e = reinterpret_cast<T *>(w);
#pragma unroll
        for (int i = 0; i < NE; ++i) e[i] = (t0 + i < L) ? row[t0 + i] : from_float<T>(0.f);
    }
}

template <int HS>
__device__ __forceinline__ void lds_pairs(const float *p, uint64_t (&v)[HS / 2])
{
    if constexpr (HS % 4 == 0) {
#pragma unroll
        for (int q = 0; q < HS / 4; ++q) {
            const ulonglong2 r = reinterpret_cast<const ulonglong2 *>(p)[q];
            v[2 * q] = r.x;
            v[2 * q + 1] = r.y;
        }
    } else {
#pragma unroll
        for (int j = 0; j < HS / 2; ++j) v[j] = reinterpret_cast<const uint64_t *>(p)[j];
    }
}

template <typename T, int NS, int W>
__global__ void __launch_bounds__(32 * W, kQuadMinBlocks) scan_quad_kernel(const mb200_scan_args a, const int vec_flags)
{
    constexpr int LPC = 4;                             // lanes per channel
    constexpr int TB = kSeqBytes / sizeof(T);          // steps per block: 16 (16-bit) or 8 (fp32)
    constexpr int HS = NS / LPC;                       // states per lane
    constexpr int HP = TB / LPC;                       // steps whose scalars this lane owns (8 bytes of a row)
    constexpr int CPW = 32 / LPC;                      // channels per warp
    constexpr int PK = 16 / sizeof(T);                 // elements of one 16-byte staging packet
    static_assert(HS % 2 == 0 && HP * sizeof(T) == 8, "lane split");
    __shared__ __align__(16) float Bs[2][TB * NS], Cs[2][TB * NS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane & (LPC - 1);                  // which quarter of the states / of the block's steps is mine
    const int N = a.dstate, L = a.seqlen;
    const int per_group = a.dim / a.ngroups;
    const int tiles_per_group = (per_group + CPW * W - 1) / (CPW * W);
    const int b = blockIdx.y;
    const int g = blockIdx.x / tiles_per_group;
    const int d = g * per_group + (blockIdx.x % tiles_per_group) * (CPW * W) + warp * CPW + (lane >> 2);
    const bool live = d < (g + 1) * per_group;
    const int dc = live ? d : g * per_group;            // idle lanes shadow a valid channel, store nothing
    const bool io_vec = vec_flags & 1, bc_vec = vec_flags & 2;

    uint64_t A2[HS / 2], h[HS / 2];
#pragma unroll
    for (int j = 0; j < HS / 2; ++j) {
        float av[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int n = sub * HS + 2 * j + e;
            av[e] = n < N ? a.A[(int64_t)dc * a.A_stride[0] + (int64_t)n * a.A_stride[1]] * kLog2e : 0.f;
        }
        A2[j] = pack2(av[0], av[1]);
        h[j] = pack2(0.f, 0.f);
    }
    const float bias = a.delta_bias ? a.delta_bias[dc] : 0.f;
    const float Dd = (a.D && sub == 0) ? a.D[dc] : 0.f;    // the skip term is added once per channel
    const T *urow = static_cast<const T *>(a.u) + (int64_t)b * a.u_stride[0] + (int64_t)dc * a.u_stride[1];
    const T *drow = static_cast<const T *>(a.delta) + (int64_t)b * a.delta_stride[0] + (int64_t)dc * a.delta_stride[1];
    const T *zrow = a.z ? static_cast<const T *>(a.z) + (int64_t)b * a.z_stride[0] + (int64_t)dc * a.z_stride[1] : nullptr;
    T *orow = static_cast<T *>(a.out) + (int64_t)b * a.out_stride[0] + (int64_t)dc * a.out_stride[1];
    T *prow = (a.z && a.out_pregate) ? static_cast<T *>(a.out_pregate) + (int64_t)b * a.pregate_stride[0] + (int64_t)dc * a.pregate_stride[1] : nullptr;

    // B/C staging: 2 tensors x NS rows x 2 packets of 16 bytes per block; thread -> (tensor, row, packet)
    const bool stager = tid < 4 * NS;
    const int st_c = tid / (2 * NS), sn = (tid % (2 * NS)) >> 1, pk = tid & 1;
    const T *ssrc = st_c ? static_cast<const T *>(a.C) + (int64_t)b * a.C_stride[0] + (int64_t)g * a.C_stride[1] + (int64_t)sn * a.C_stride[2]
                         : static_cast<const T *>(a.B) + (int64_t)b * a.B_stride[0] + (int64_t)g * a.B_stride[1] + (int64_t)sn * a.B_stride[2];
    auto stage_load = [&](int t0) {
        uint4 r = make_uint4(0, 0, 0, 0);
        const int ts = t0 + pk * PK;
        if (stager && sn < N) {
            if (bc_vec && ts + PK <= L) {
                r = *reinterpret_cast<const uint4 *>(ssrc + ts);
            } else {
                T *e = reinterpret_cast<T *>(&r);
#pragma unroll
                for (int i = 0; i < PK; ++i) e[i] = (ts + i < L) ? ssrc[ts + i] : from_float<T>(0.f);
            }
        }
        return r;
    };
    auto stage_store = [&](int buf, const uint4 &r) {
        if (stager) {
            float *dst = st_c ? Cs[buf] : Bs[buf];
            const T *e = reinterpret_cast<const T *>(&r);
#pragma unroll
            for (int i = 0; i < PK; ++i) dst[(pk * PK + i) * NS + sn] = to_float(e[i]);
        }
    };

    const int nblk = (L + TB - 1) / TB;
    stage_store(0, stage_load(0));
    uint32_t ru[kSeqBytes / 4], rd[2];
    for (int blk = 0; blk < nblk; ++blk) {
        const int t0 = blk * TB, buf = blk & 1;
        const int ts = t0 + sub * HP;                   // first of my own steps
        __syncthreads();            // tile of this block in place; every warp is done with the other buffer
        uint4 nbc = make_uint4(0, 0, 0, 0);
        if (blk + 1 < nblk) nbc = stage_load(t0 + TB);
        row_load<T, kSeqBytes>(ru, urow, t0, L, io_vec);
        row_load<T, 8>(rd, drow, ts, L, io_vec);
        uint32_t rz[2] = {0u, 0u};
        if (zrow) row_load<T, 8>(rz, zrow, ts, L, io_vec);
        {   // sectors of a later block start moving while this block is computed
            const int tp = t0 + kSeqAhead * TB;
            seq_prefetch(urow, tp, L);
            seq_prefetch(drow, tp + sub * HP, L);
            if (zrow) seq_prefetch(zrow, tp + sub * HP, L);
            if (stager && sn < N) seq_prefetch(ssrc, tp + pk * PK, L);
        }
        float dtm[HP];
#pragma unroll
        for (int i = 0; i < HP; ++i) {
            float v = words_get<T>(rd, i) + bias;
            if (a.delta_softplus) v = fast_softplus20(v);
            if (ts + i >= L) v = 0.f;                   // steps past the end are the identity (1, 0)
            dtm[i] = v;
        }
        const float *Bt = Bs[buf] + sub * HS, *Ct = Cs[buf] + sub * HS;
        float ym[HP];
#pragma unroll
        for (int i = 0; i < TB; ++i) {
            const float uu = words_get<T>(ru, i);
            const float dl = __shfl_sync(0xffffffffu, dtm[i % HP], (lane & ~(LPC - 1)) | (i / HP));
            const float du = dl * uu;
            const uint64_t dl2 = pack2(dl, dl), du2 = pack2(du, du);
            uint64_t bp[HS / 2], cp[HS / 2];
            lds_pairs<HS>(Bt + i * NS, bp);
            lds_pairs<HS>(Ct + i * NS, cp);
            uint64_t ya = pack2(Dd * uu, 0.f);
#pragma unroll
            for (int j = 0; j < HS / 2; ++j) {
                float x0, x1;
                unpack2(mul2(dl2, A2[j]), x0, x1);
                h[j] = fma2(pack2(ex2(x0), ex2(x1)), h[j], mul2(du2, bp[j]));
                ya = fma2(h[j], cp[j], ya);
            }
            float s0, s1;
            unpack2(ya, s0, s1);
            float y = s0 + s1;
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            y += __shfl_xor_sync(0xffffffffu, y, 2);
            if (sub == i / HP) ym[i % HP] = y;
        }
        if (live) {
            float yg[HP];
#pragma unroll
            for (int i = 0; i < HP; ++i) {
                if (zrow) {
                    const float zz = words_get<T>(rz, i);
                    if constexpr (std::is_same<T, __nv_bfloat16>::value) yg[i] = ym[i] * silu_for_bf16(zz);
                    else yg[i] = ym[i] * fast_silu(zz);
                } else {
                    yg[i] = ym[i];
                }
            }
            auto put = [&](T *row, const float (&v)[HP]) {
                if (io_vec && ts + HP <= L) {
                    uint2 o;
                    T *e = reinterpret_cast<T *>(&o);
#pragma unroll
                    for (int i = 0; i < HP; ++i) e[i] = from_float<T>(v[i]);
                    *reinterpret_cast<uint2 *>(row + ts) = o;
                } else {
#pragma unroll
                    for (int i = 0; i < HP; ++i)
                        if (ts + i < L) row[ts + i] = from_float<T>(v[i]);
                }
            };
            put(orow, yg);
            if (prow) put(prow, ym);
        }
        if (blk + 1 < nblk) stage_store(buf ^ 1, nbc);
    }
    if (a.last_state && live) {
        float *ls = a.last_state + ((int64_t)b * a.dim + d) * N;
#pragma unroll
        for (int j = 0; j < HS / 2; ++j) {
            float lo, hi;
            unpack2(h[j], lo, hi);
            if (sub * HS + 2 * j < N) ls[sub * HS + 2 * j] = lo;
            if (sub * HS + 2 * j + 1 < N) ls[sub * HS + 2 * j + 1] = hi;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Warp-specialised variant of the channel-parallel scan (dstate <= 16, input-dependent B and C,
// 16-byte aligned rows).  The lanes of a warp are 32 different CHANNELS, so B_t and C_t are read
// from shared memory at one address per warp (a single wavefront per 128-bit load), and nothing in
// the recurrence loop crosses lanes.  A CTA of three warps owns 32 channels of one batch row:
//   warp 0   ("scalar" warp) streams the u, dt, z rows and the group's B/C rows as TMA tiles
//            (32 bytes of every row per tile, SWIZZLE_32B so that each lane reads its own row without
//            bank conflicts), evaluates softplus(dt) and hands (dt, u) for 8 steps at a time to the
//            state warps through shared memory (dt and dt*u) together with the B/C values converted to
//            fp32; later it adds the two partial outputs and D*u, applies silu(z) and sends the output
//            tile back with a TMA store;
//   warps 1,2 ("state" warps) each keep half of the states of the 32 channels in registers and run
//            the recurrence: per (step, state) one MUFU ex2 and four FMA-pipe operations, no shuffles.
// Hand-offs are mbarriers: ready[2] (scalar -> state, 8 steps of dt/u/B/C in place) and ydone[2]
// (state -> scalar, 8 steps of partial outputs in place), all buffers double.  The scalar warp runs
// one hand-off ahead, and the TMA tiles two tiles ahead, of the recurrence.  Every wait is bounded;
// on expiry the kernel records a code in g_scan_status, stops, and drains its outstanding copies.
__device__ int g_scan_status;
enum { kStScanFull = 31, kStScanZ, kStScanReady, kStScanYdone, kStScanAlign };

constexpr int kStreamCh = 32;      // channels per CTA (lanes of a warp)
constexpr int64_t kStreamMinChannels = 1024;   // fewer (batch x dim) channels than this go to the time-parallel kernel
constexpr int kHB = 8;             // steps per hand-off

struct ScanMaps { CUtensorMap u, dt, z, out, B, C; };

// Sequence split inside one launch: CTA (group of channels, batch row, segment) walks steps [s * seg_len, (s+1) * seg_len)
// from the state h0[b][s] (zero when h0 is NULL).  A SUMMARY launch computes, for every segment but the last, the state
// at its end from a zero start (hend) and the product of its decays (pdec); after a fold over the segments a second,
// full launch runs every segment from its true entering state.  nseg = 1 is the plain one-pass scan.
struct ScanSplit {
    int nseg, seg_len;
    const float *h0;        // (batch, nseg, dim, dstate) or NULL
    float *hend, *pdec;     // (batch, nseg, dim, dstate), SUMMARY launches only
};

template <typename T, int NS, int SW, int NB>
struct __align__(256) StreamSmem {
    uint8_t u[2][kStreamCh * 32];
    uint8_t dt[2][kStreamCh * 32];
    uint8_t z[2][kStreamCh * 32];
    uint8_t out[2][kStreamCh * 32];
    uint8_t B[2][(NS * 32 + 255) / 256 * 256];
    uint8_t C[2][(NS * 32 + 255) / 256 * 256];
    // per-channel rows of 8 steps (32 bytes) in the same chunk-swizzled layout as the tiles: a lane moves four
    // steps with one conflict-free 128-bit access
    float xd[NB][2][kStreamCh * kHB];        // [buffer][dt | dt*u][channel][step]
    float du[NB][kStreamCh * kHB];           // [buffer][channel][step]: D*u, kept by the scalar warp for its epilogue
    float bc[NB][2][kHB * NS + 16];          // [buffer][B | C][step][state]; the pad puts B and C on different banks
    float yp[NB][SW][kStreamCh * kHB];       // [buffer][state warp][channel][step]
    uint64_t full[2], zfull[2], ready[NB], ydone[NB], edone[NB];
};

// byte offset of 16-byte chunk `chunk` of row `row` in a [rows x 32 B] SWIZZLE_32B tile (256-byte aligned)
__device__ __forceinline__ int sw32_offset(int row, int chunk) { return row * 32 + ((chunk ^ ((row >> 2) & 1)) << 4); }

// SW state warps share the states of the 32 channels; SPLIT gives the scalar work to two warps (warp 0 streams the
// tiles in and prepares the hand-offs, warp 1 finishes the outputs and streams them out) instead of one.  (2, false) is
// the layout described above: three warps, nine CTAs per SM, the choice whenever the grid fills the GPU.  The other two
// are for grids that leave the SMs partly empty (a batch divided over several GPUs), where a CTA's own serial chain per
// hand-off matters more than the number of CTAs an SM can hold: (2, true), four warps and six CTAs per SM, for up to
// 888 CTAs; (4, true), six warps (four states per lane) and four CTAs per SM, for up to 592.
template <typename T, int NS, bool SUMMARY, int SW, bool SPLIT>
__global__ void __launch_bounds__(32 * (SW + (SPLIT ? 2 : 1)), !SPLIT ? 9 : SW == 2 ? 6 : 4)
scan_stream_kernel(const mb200_scan_args a, const __grid_constant__ ScanMaps maps, const ScanSplit sp)
{
    using namespace tc;
    constexpr int TB = 32 / sizeof(T);                 // steps per tile (32 bytes of a row)
    constexpr int HPT = TB / kHB;                      // hand-offs per tile: 2 (16-bit) or 1 (fp32)
    constexpr int CPH = kHB * sizeof(T) / 16;          // 16-byte chunks per hand-off: 1 or 2
    constexpr int HS = NS / SW;                        // states per lane of a state warp
    constexpr int kScalarWarps = SPLIT ? 2 : 1;
    // hand-off buffers: with one scalar warp two are all it can use (it prepares hand-off hb+1, then finishes hb); with
    // the work on two warps, four let the three stages of the chain run at the pace of the slowest, not of their sum
    constexpr int NB = SPLIT ? 4 : 2;
    extern __shared__ __align__(256) uint8_t smem_raw[];
    StreamSmem<T, NS, SW, NB> &sm = *reinterpret_cast<StreamSmem<T, NS, SW, NB> *>(smem_raw);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int N = a.dstate;
    const int b = blockIdx.y / sp.nseg, seg = blockIdx.y % sp.nseg;
    const int t_begin = seg * sp.seg_len;              // a multiple of the tile length
    const int L = min(a.seqlen, t_begin + sp.seg_len) - t_begin;      // steps of my segment
    const int ch0 = blockIdx.x * kStreamCh;
    const int d = ch0 + lane;                          // my channel (dim is a multiple of 32 on this path)
    const int g = ch0 / (a.dim / a.ngroups);
    const int ntiles = (L + TB - 1) / TB, nhb = (L + kHB - 1) / kHB;
    const bool has_z = !SUMMARY && a.z != nullptr;
    if (SUMMARY && seg == sp.nseg - 1) return;         // the last segment's end state is the full launch's business
    if (L <= 0) return;                                // a segment past the end of a short sequence
    int *status = &g_scan_status;
    if (smem_u32(smem_raw) & 255u) {                   // the swizzle pattern of the tiles assumes this alignment
        if (threadIdx.x == 0) atomicCAS(status, 0, kStScanAlign);
        return;
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&sm.full[i], 1);
            mbar_init(&sm.zfull[i], 1);
        }
        for (int i = 0; i < NB; ++i) {
            mbar_init(&sm.ready[i], 1);
            mbar_init(&sm.ydone[i], SW);
            mbar_init(&sm.edone[i], 1);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp < kScalarWarps) {
        // ------------------------------------------------------------------ scalar warp(s)
        const bool in_side = warp == 0, out_side = warp == kScalarWarps - 1;
        constexpr uint32_t kTileBytes = 2 * kStreamCh * 32 + (SUMMARY ? 1 : 2) * NS * 32;      // a summary needs no C
        auto issue_tile = [&](int k) {          // lane 0 only
            const int s = k & 1;
            mbar_expect_tx(&sm.full[s], kTileBytes);
            tma_load_3d(sm.u[s], &maps.u, &sm.full[s], t_begin + k * TB, ch0, b);
            tma_load_3d(sm.dt[s], &maps.dt, &sm.full[s], t_begin + k * TB, ch0, b);
            tma_load_4d(sm.B[s], &maps.B, &sm.full[s], t_begin + k * TB, 0, g, b);
            if (!SUMMARY) tma_load_4d(sm.C[s], &maps.C, &sm.full[s], t_begin + k * TB, 0, g, b);
        };
        auto issue_z = [&](int k) {             // lane 0 only
            const int s = k & 1;
            mbar_expect_tx(&sm.zfull[s], kStreamCh * 32);
            tma_load_3d(sm.z[s], &maps.z, &sm.zfull[s], t_begin + k * TB, ch0, b);
        };
        int issued = 0, zissued = 0, waited = 0, zwaited = 0;     // tiles requested / consumed (uniform across the warp)
        if (lane == 0) {
            prefetch_tmap(&maps.u); prefetch_tmap(&maps.dt); prefetch_tmap(&maps.B);
            if (!SUMMARY) { prefetch_tmap(&maps.C); prefetch_tmap(&maps.out); }
            if (has_z) prefetch_tmap(&maps.z);
        }
        for (int k = 0; k < 2 && k < ntiles; ++k) {
            if (lane == 0 && in_side) issue_tile(k);
            if (lane == 0 && out_side && has_z) issue_z(k);
            ++issued; ++zissued;
        }
        const float bias = a.delta_bias ? a.delta_bias[d] : 0.f;
        const float Dd = a.D ? a.D[d] : 0.f;
        const int st_t = lane / NS, st_n = lane % NS;     // my (tensor, state row) in the B/C conversion
        const bool st_on = lane < (SUMMARY ? 1 : 2) * NS;
        bool ok = true;

        auto prologue = [&](int hb) {
            const int k = hb / HPT, s = k & 1, part = hb % HPT, buf = hb % NB;
            if (SPLIT && hb >= NB) {    // the other scalar warp has finished with this buffer's D*u and partial outputs
                if (!mbar_wait(&sm.edone[buf], ((hb - NB) / NB) & 1, status, kStScanYdone)) { ok = false; return; }
            }
            if (part == 0) {
                if (!mbar_wait(&sm.full[s], (k >> 1) & 1, status, kStScanFull)) { ok = false; return; }
                ++waited;
            }
            uint32_t wd[CPH * 4], wu[CPH * 4];
#pragma unroll
            for (int c = 0; c < CPH; ++c) {
                const int off = sw32_offset(lane, part * CPH + c);
                const uint4 rd = *reinterpret_cast<const uint4 *>(sm.dt[s] + off);
                const uint4 ru = *reinterpret_cast<const uint4 *>(sm.u[s] + off);
                wd[4 * c] = rd.x; wd[4 * c + 1] = rd.y; wd[4 * c + 2] = rd.z; wd[4 * c + 3] = rd.w;
                wu[4 * c] = ru.x; wu[4 * c + 1] = ru.y; wu[4 * c + 2] = ru.z; wu[4 * c + 3] = ru.w;
            }
            uint32_t wb[CPH * 4];
            if (st_on) {
                const uint8_t *src = st_t ? sm.C[s] : sm.B[s];
#pragma unroll
                for (int c = 0; c < CPH; ++c) {
                    const uint4 r = *reinterpret_cast<const uint4 *>(src + sw32_offset(st_n, part * CPH + c));
                    wb[4 * c] = r.x; wb[4 * c + 1] = r.y; wb[4 * c + 2] = r.z; wb[4 * c + 3] = r.w;
                }
            }
            const int t0 = hb * kHB;
            const bool tail = t0 + kHB > L;             // only the last hand-off can run past the end
            float dl[kHB], dlu[kHB], skip[kHB];
#pragma unroll
            for (int i = 0; i < kHB; ++i) {
                float v = words_get<T>(wd, i) + bias;
                if (a.delta_softplus) v = sizeof(T) == 2 ? softplus20_lowprec(v) : fast_softplus20(v);
                if (tail && t0 + i >= L) v = 0.f;       // steps past the end are the identity (1, 0)
                const float uu = words_get<T>(wu, i);
                dl[i] = v;
                dlu[i] = v * uu;
                skip[i] = Dd * uu;
            }
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int off = sw32_offset(lane, c);
                *reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(sm.xd[buf][0]) + off) = make_float4(dl[4 * c], dl[4 * c + 1], dl[4 * c + 2], dl[4 * c + 3]);
                *reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(sm.xd[buf][1]) + off) = make_float4(dlu[4 * c], dlu[4 * c + 1], dlu[4 * c + 2], dlu[4 * c + 3]);
                *reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(sm.du[buf]) + off) = make_float4(skip[4 * c], skip[4 * c + 1], skip[4 * c + 2], skip[4 * c + 3]);
            }
            if (st_on) {
                float *dst = sm.bc[buf][st_t];
#pragma unroll
                for (int i = 0; i < kHB; ++i) dst[i * NS + st_n] = words_get<T>(wb, i);
            }
            __syncwarp();
            if (lane == 0) {
                if ((part == HPT - 1 || hb == nhb - 1) && k + 2 < ntiles) issue_tile(k + 2);
                mbar_arrive(&sm.ready[buf]);
            }
            if ((part == HPT - 1 || hb == nhb - 1) && k + 2 < ntiles) ++issued;
        };

        auto epilogue = [&](int hb) {
            const int k = hb / HPT, s = k & 1, part = hb % HPT, buf = hb % NB;
            if (!mbar_wait(&sm.ydone[buf], (hb / NB) & 1, status, kStScanYdone)) { ok = false; return; }
            if (SUMMARY) {                      // nothing to put out: the wait only hands the buffers back
                if (SPLIT && lane == 0) mbar_arrive(&sm.edone[buf]);
                return;
            }
            if (part == 0) {
                if (has_z) {
                    if (!mbar_wait(&sm.zfull[s], (k >> 1) & 1, status, kStScanZ)) { ok = false; return; }
                    ++zwaited;
                }
                if (k >= 2) {       // the store that last read this output tile has finished reading it
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    __syncwarp();
                }
            }
            float y[kHB];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int off = sw32_offset(lane, c);
                float4 p0 = *reinterpret_cast<const float4 *>(reinterpret_cast<const uint8_t *>(sm.yp[buf][0]) + off);
                const float4 p1 = *reinterpret_cast<const float4 *>(reinterpret_cast<const uint8_t *>(sm.yp[buf][1]) + off);
                if constexpr (SW == 4) {
                    const float4 p2 = *reinterpret_cast<const float4 *>(reinterpret_cast<const uint8_t *>(sm.yp[buf][2]) + off);
                    const float4 p3 = *reinterpret_cast<const float4 *>(reinterpret_cast<const uint8_t *>(sm.yp[buf][3]) + off);
                    p0 = make_float4(p0.x + p2.x, p0.y + p2.y, p0.z + p2.z, p0.w + p2.w);
                    p0 = make_float4(p0.x + p3.x, p0.y + p3.y, p0.z + p3.z, p0.w + p3.w);
                }
                const float4 sk = *reinterpret_cast<const float4 *>(reinterpret_cast<const uint8_t *>(sm.du[buf]) + off);
                y[4 * c] = (p0.x + p1.x) + sk.x;
                y[4 * c + 1] = (p0.y + p1.y) + sk.y;
                y[4 * c + 2] = (p0.z + p1.z) + sk.z;
                y[4 * c + 3] = (p0.w + p1.w) + sk.w;
            }
            if (SPLIT) {        // D*u and the partial outputs of this buffer are in registers: the other warp may refill it
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.edone[buf]);
            }
            if (has_z) {
                uint32_t wz[CPH * 4];
#pragma unroll
                for (int c = 0; c < CPH; ++c) {
                    const uint4 r = *reinterpret_cast<const uint4 *>(sm.z[s] + sw32_offset(lane, part * CPH + c));
                    wz[4 * c] = r.x; wz[4 * c + 1] = r.y; wz[4 * c + 2] = r.z; wz[4 * c + 3] = r.w;
                }
#pragma unroll
                for (int i = 0; i < kHB; ++i) {
                    const float zz = words_get<T>(wz, i);
                    if constexpr (std::is_same<T, __nv_bfloat16>::value) y[i] *= silu_for_bf16(zz);
                    else y[i] *= fast_silu(zz);
                }
            }
            uint32_t wo[CPH * 4];
            {
                T *e = reinterpret_cast<T *>(wo);
#pragma unroll
                for (int i = 0; i < kHB; ++i) e[i] = from_float<T>(y[i]);
            }
#pragma unroll
            for (int c = 0; c < CPH; ++c)
                *reinterpret_cast<uint4 *>(sm.out[s] + sw32_offset(lane, part * CPH + c)) =
                    make_uint4(wo[4 * c], wo[4 * c + 1], wo[4 * c + 2], wo[4 * c + 3]);
            if (part == HPT - 1 || hb == nhb - 1) {
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(&maps.out),
                                 "r"(smem_u32(sm.out[s])), "r"(t_begin + k * TB), "r"(ch0), "r"(b)
                                 : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    if (has_z && k + 2 < ntiles) issue_z(k + 2);
                }
                if (has_z && k + 2 < ntiles) ++zissued;
            }
        };

        if (!SPLIT) {
            prologue(0);
            for (int hb = 0; hb < nhb && ok; ++hb) {
                if (hb + 1 < nhb) prologue(hb + 1);
                if (ok) epilogue(hb);
            }
        } else if (in_side) {
            for (int hb = 0; hb < nhb && ok; ++hb) prologue(hb);
        } else {
            for (int hb = 0; hb < nhb && ok; ++hb) epilogue(hb);
        }
        if (lane == 0) {
            if (out_side) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            if (!ok) {      // stopped early: let the tiles already requested land before the CTA's shared memory goes away
                if (in_side)
                    for (int k = waited; k < issued; ++k) mbar_wait(&sm.full[k & 1], (k >> 1) & 1, status, kStScanFull);
                if (out_side && has_z)
                    for (int k = zwaited; k < zissued; ++k) mbar_wait(&sm.zfull[k & 1], (k >> 1) & 1, status, kStScanZ);
            }
        }
    } else {
        // ------------------------------------------------------------------ state warps
        const int w = warp - kScalarWarps;
        uint64_t A2[HS / 2], h[HS / 2];
#pragma unroll
        for (int j = 0; j < HS / 2; ++j) {
            float av[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = w * HS + 2 * j + e;
                av[e] = n < N ? a.A[(int64_t)d * a.A_stride[0] + (int64_t)n * a.A_stride[1]] * kLog2e : 0.f;
            }
            A2[j] = pack2(av[0], av[1]);
            float h0v[2] = {0.f, 0.f};
            if (sp.h0) {
                const float *hp = sp.h0 + (((int64_t)b * sp.nseg + seg) * a.dim + d) * N;
#pragma unroll
                for (int e = 0; e < 2; ++e)
                    if (w * HS + 2 * j + e < N) h0v[e] = hp[w * HS + 2 * j + e];
            }
            h[j] = pack2(h0v[0], h0v[1]);
        }
        float sum_dl = 0.f;          // SUMMARY: the decay product of the segment is 2^(A log2e * sum of dt)
        for (int hb = 0; hb < nhb; ++hb) {
            const int buf = hb % NB;
            if (!mbar_wait(&sm.ready[buf], (hb / NB) & 1, status, kStScanReady)) break;
            const float *Bt = sm.bc[buf][0] + w * HS, *Ct = sm.bc[buf][1] + w * HS;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int off = sw32_offset(lane, c);
                const float4 dlv = *reinterpret_cast<const float4 *>(reinterpret_cast<const uint8_t *>(sm.xd[buf][0]) + off);
                const float4 duv = *reinterpret_cast<const float4 *>(reinterpret_cast<const uint8_t *>(sm.xd[buf][1]) + off);
                const float dls[4] = {dlv.x, dlv.y, dlv.z, dlv.w}, dus[4] = {duv.x, duv.y, duv.z, duv.w};
                float ys[4];
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const int i = 4 * c + i4;
                    const uint64_t dl2 = pack2(dls[i4], dls[i4]), du2 = pack2(dus[i4], dus[i4]);
                    uint64_t bp[HS / 2], cp[HS / 2];
                    lds_pairs<HS>(Bt + i * NS, bp);
                    if (SUMMARY) {
                        sum_dl += dls[i4];
#pragma unroll
                        for (int j = 0; j < HS / 2; ++j) {
                            float x0, x1;
                            unpack2(mul2(dl2, A2[j]), x0, x1);
                            h[j] = fma2(pack2(ex2(x0), ex2(x1)), h[j], mul2(du2, bp[j]));
                        }
                        ys[i4] = 0.f;
                    } else {
                        lds_pairs<HS>(Ct + i * NS, cp);
                        uint64_t ya = pack2(0.f, 0.f), yb = pack2(0.f, 0.f);
#pragma unroll
                        for (int j = 0; j < HS / 2; ++j) {
                            float x0, x1;
                            unpack2(mul2(dl2, A2[j]), x0, x1);
                            h[j] = fma2(pack2(ex2(x0), ex2(x1)), h[j], mul2(du2, bp[j]));
                            if (j & 1) yb = fma2(h[j], cp[j], yb);
                            else ya = fma2(h[j], cp[j], ya);
                        }
                        float s0, s1, s2, s3;
                        unpack2(ya, s0, s1);
                        unpack2(yb, s2, s3);
                        ys[i4] = (s0 + s1) + (s2 + s3);
                    }
                }
                if (!SUMMARY) *reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(sm.yp[buf][w]) + off) = make_float4(ys[0], ys[1], ys[2], ys[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.ydone[buf]);
        }
        if (SUMMARY) {
            const int64_t o = (((int64_t)b * sp.nseg + seg) * a.dim + d) * N;
#pragma unroll
            for (int j = 0; j < HS / 2; ++j) {
                float lo, hi, a0, a1;
                unpack2(h[j], lo, hi);
                unpack2(A2[j], a0, a1);
                const int n = w * HS + 2 * j;
                if (n < N) { sp.hend[o + n] = lo; sp.pdec[o + n] = ex2(a0 * sum_dl); }
                if (n + 1 < N) { sp.hend[o + n + 1] = hi; sp.pdec[o + n + 1] = ex2(a1 * sum_dl); }
            }
        } else if (a.last_state && seg == sp.nseg - 1) {
            float *ls = a.last_state + ((int64_t)b * a.dim + d) * N;
#pragma unroll
            for (int j = 0; j < HS / 2; ++j) {
                float lo, hi;
                unpack2(h[j], lo, hi);
                if (w * HS + 2 * j < N) ls[w * HS + 2 * j] = lo;
                if (w * HS + 2 * j + 1 < N) ls[w * HS + 2 * j + 1] = hi;
            }
        }
    }
}

// h0[b][s+1] = pdec[b][s] * h0[b][s] + hend[b][s] over the segments of a split sequence, one thread per (row, channel, state)
__global__ void __launch_bounds__(256) scan_fold_segments_kernel(float *h0, const float *hend, const float *pdec, int nseg, int64_t per_seg,
                                                                 int64_t rows)
{
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= rows * per_seg) return;
    const int64_t b = i / per_seg, e = i % per_seg;
    float h = 0.f;
    for (int s = 0; s < nseg; ++s) {
        const int64_t o = (b * nseg + s) * per_seg + e;
        h0[o] = h;
        if (s + 1 < nseg) h = fmaf(pdec[o], h, hend[o]);
    }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T> int split_segments(const mb200_scan_args &a);

// The warp-specialised kernel needs TMA-describable operands: 16-byte aligned bases and row strides, whole
// groups of 32 channels, input-dependent B and C, and no separate pre-gate output.
template <typename T>
bool stream_eligible(const mb200_scan_args &a)
{
    constexpr int VEC = 16 / sizeof(T);
    if (a.dstate > 16 || !a.B_variable || !a.C_variable || a.out_pregate) return false;
    if ((a.dim / a.ngroups) % kStreamCh != 0) return false;
    // the output tile store clips the innermost dimension in 16-byte units, not in elements: a row (of a wider buffer)
    // that ends inside such a unit would have the bytes after its end overwritten
    if (((size_t)a.seqlen * sizeof(T)) % 16 != 0) return false;
    if ((int64_t)a.batch * a.dim < kStreamMinChannels && split_segments<T>(a) <= 1) return false;
    auto ok2 = [&](const void *p, const int64_t *s) { return aligned16(p) && s[0] > 0 && s[1] > 0 && s[0] % VEC == 0 && s[1] % VEC == 0; };
    auto ok3 = [&](const void *p, const int64_t *s) {
        return aligned16(p) && s[0] > 0 && s[1] > 0 && s[2] > 0 && s[0] % VEC == 0 && s[1] % VEC == 0 && s[2] % VEC == 0;
    };
    if (!ok2(a.u, a.u_stride) || !ok2(a.delta, a.delta_stride) || !ok2(a.out, a.out_stride)) return false;
    if (a.z && !ok2(a.z, a.z_stride)) return false;
    if (!ok3(a.B, a.B_stride) || !ok3(a.C, a.C_stride)) return false;
    return encode_fn() != nullptr;
}

// How many segments the sequence is cut into (1 = one pass).  Cutting pays when the channel groups alone leave most
// of the GPU idle: with G = batch * dim / 32 groups, nseg is the largest power of two with G * nseg CTAs in one wave
// of 9 per SM.  It costs a second pass over every segment but the last, so it is used only from nseg = 8 up (fewer
// segments measured no faster than one pass), with segments of at least 128 steps, and only when the caller lent
// scratch for the summaries.
template <typename T>
int split_segments(const mb200_scan_args &a)
{
    const int64_t groups = (int64_t)a.batch * a.dim / kStreamCh;
    if (groups <= 0) return 1;
    int nseg = 1;
    while (nseg < 16 && groups * nseg * 2 <= 9 * 148 && a.seqlen / (nseg * 2) >= 128) nseg *= 2;
    if (nseg < 8) return 1;
    const size_t need = 3 * sizeof(float) * (size_t)a.batch * nseg * a.dim * a.dstate;
    if (!a.scratch || a.scratch_bytes < need || (reinterpret_cast<uintptr_t>(a.scratch) & 15)) return 1;
    return nseg;
}

template <typename T>
int launch_stream(const mb200_scan_args &a, cudaStream_t stream)
{
    constexpr uint32_t TB = 32 / sizeof(T);
    const int dtype = sizeof(T) == 4 ? MB200_F32 : (std::is_same<T, __half>::value ? MB200_F16 : MB200_BF16);
    ScanMaps maps;
    auto rows = [&](CUtensorMap *m, const void *p, const int64_t *st) {
        const uint64_t dims[3] = {(uint64_t)a.seqlen, (uint64_t)a.dim, (uint64_t)a.batch};
        const uint64_t sb[2] = {(uint64_t)st[1] * sizeof(T), (uint64_t)st[0] * sizeof(T)};
        const uint32_t box[3] = {TB, (uint32_t)kStreamCh, 1};
        return encode_tiled(m, dtype, p, 3, dims, sb, box, CU_TENSOR_MAP_SWIZZLE_32B);
    };
    auto bc = [&](CUtensorMap *m, const void *p, const int64_t *st, uint32_t ns) {
        const uint64_t dims[4] = {(uint64_t)a.seqlen, (uint64_t)a.dstate, (uint64_t)a.ngroups, (uint64_t)a.batch};
        const uint64_t sb[3] = {(uint64_t)st[2] * sizeof(T), (uint64_t)st[1] * sizeof(T), (uint64_t)st[0] * sizeof(T)};
        const uint32_t box[4] = {TB, ns, 1, 1};
        return encode_tiled(m, dtype, p, 4, dims, sb, box, CU_TENSOR_MAP_SWIZZLE_32B);
    };
    const uint32_t ns = a.dstate <= 8 ? 8 : 16;
    bool ok = rows(&maps.u, a.u, a.u_stride) && rows(&maps.dt, a.delta, a.delta_stride) && rows(&maps.out, a.out, a.out_stride) &&
              bc(&maps.B, a.B, a.B_stride, ns) && bc(&maps.C, a.C, a.C_stride, ns);
    if (a.z) ok = ok && rows(&maps.z, a.z, a.z_stride);
    else maps.z = maps.u;
    if (!ok) return 1;      // the driver refused a map (unusual strides): the caller uses the register-staged kernel
    int nseg = split_segments<T>(a);
    int seg_len = (int)((a.seqlen + TB - 1) / TB * TB);
    if (nseg > 1) {
        seg_len = (int)(((a.seqlen + nseg - 1) / nseg + TB - 1) / TB * TB);     // whole tiles per segment
        nseg = (a.seqlen + seg_len - 1) / seg_len;                              // rounding up may leave the last ones empty
    }
    // A grid that leaves the SMs partly empty runs the six- or four-warp layout (four / six CTAs of them fit an SM).
    auto go = [&](dim3 grid, const ScanSplit &split, bool summary) {
        const int64_t ctas = (int64_t)grid.x * grid.y;
        auto pick = [&](auto ns_c, auto sum_c) {
            constexpr int NS = decltype(ns_c)::value;
            constexpr bool SUM = decltype(sum_c)::value;
            if (ctas <= 4 * 148) scan_stream_kernel<T, NS, SUM, 4, true><<<grid, 192, sizeof(StreamSmem<T, NS, 4, 4>), stream>>>(a, maps, split);
            else if (ctas <= 6 * 148) scan_stream_kernel<T, NS, SUM, 2, true><<<grid, 128, sizeof(StreamSmem<T, NS, 2, 4>), stream>>>(a, maps, split);
            else scan_stream_kernel<T, NS, SUM, 2, false><<<grid, 96, sizeof(StreamSmem<T, NS, 2, 2>), stream>>>(a, maps, split);
        };
        if (ns == 8) summary ? pick(std::integral_constant<int, 8>{}, std::true_type{}) : pick(std::integral_constant<int, 8>{}, std::false_type{});
        else summary ? pick(std::integral_constant<int, 16>{}, std::true_type{}) : pick(std::integral_constant<int, 16>{}, std::false_type{});
    };
    if (nseg <= 1) {
        const ScanSplit one = {1, seg_len, nullptr, nullptr, nullptr};
        go(dim3(a.dim / kStreamCh, a.batch), one, false);
        return MB200_OK;
    }
    // Few channel groups: the sequence is cut into nseg segments that run side by side.  A first launch summarises
    // every segment but the last from a zero state (end state + decay product), a fold turns the summaries into the
    // state entering each segment, a second launch runs every segment from there.
    const int64_t per_seg = (int64_t)a.dim * a.dstate, region = (int64_t)a.batch * nseg * per_seg;
    float *h0 = static_cast<float *>(a.scratch), *hend = h0 + region, *pdec = hend + region;
    const ScanSplit sum = {nseg, seg_len, nullptr, hend, pdec}, full = {nseg, seg_len, h0, nullptr, nullptr};
    dim3 grid(a.dim / kStreamCh, a.batch * nseg);       // in the summary launch the CTAs of the last segment return at once
    go(grid, sum, true);
    scan_fold_segments_kernel<<<(unsigned)((a.batch * per_seg + 255) / 256), 256, 0, stream>>>(h0, hend, pdec, nseg, per_seg, a.batch);
    go(grid, full, false);
    return MB200_OK;
}

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
    if (stream_eligible<T>(a)) {
        const int rc = launch_stream<T>(a, stream);
        if (rc <= 0) return rc;
    }
    // Enough independent channels to give every SM a few warps: four lanes per channel, time sequential.
    if (N <= 16 && a.B_variable && a.C_variable && (int64_t)a.batch * a.dim >= 2LL * 32 * 148) {
        // the B/C tile is fetched in 16-byte packets here
        const bool bc16 = bc_vec && aligned16(a.B) && aligned16(a.C) && a.B_stride[0] % VEC == 0 && a.B_stride[1] % VEC == 0 &&
                          a.B_stride[2] % VEC == 0 && a.C_stride[0] % VEC == 0 && a.C_stride[1] % VEC == 0 && a.C_stride[2] % VEC == 0;
        const int flags = (io_vec ? 1 : 0) | (bc16 ? 2 : 0);
        constexpr int QW = kQuadWarps;
        dim3 grid(a.ngroups * ((per_group + 8 * QW - 1) / (8 * QW)), a.batch);
        if (N <= 8) scan_quad_kernel<T, 8, QW><<<grid, 32 * QW, 0, stream>>>(a, flags);
        else scan_quad_kernel<T, 16, QW><<<grid, 32 * QW, 0, stream>>>(a, flags);
        return MB200_OK;
    }
    const size_t smem = sizeof(float) * (2 * kStateBlock * kTile + 2 * (size_t)chans * npad);
    static_assert(2 * kStateBlock * kTile * sizeof(float) + 2 * kWarps * 2 * 256 * sizeof(float) <= 227 * 1024, "smem budget");
    cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(&scan_fwd_kernel<T>), (int)smem, a.device);
    if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "selective_scan: shared memory opt-in (%zu B): %s", smem, cudaGetErrorString(e));
    const int tiles_per_group = (per_group + chans - 1) / chans;
    dim3 grid(a.ngroups * tiles_per_group, a.batch);
    scan_fwd_kernel<T><<<grid, kThreads, smem, stream>>>(a, cpw, nblocks, npad, vec_flags);
    return MB200_OK;
}

}  // namespace
}  // namespace mb200

extern "C" int mb200_scan_scratch_bytes(const mb200_scan_args *args, size_t *bytes)
{
    using namespace mb200;
    if (!args || !bytes) return fail(MB200_ERR_BAD_ARG, "scan_scratch_bytes: NULL argument");
    const mb200_scan_args &a = *args;
    *bytes = 0;
    if (a.batch <= 0 || a.dim <= 0 || a.dstate <= 0 || a.dstate > 16 || a.seqlen <= 0) return MB200_OK;
    // the size that would let the sequence be cut: ask the policy with a scratch that is certainly large enough
    mb200_scan_args probe = a;
    probe.scratch = reinterpret_cast<void *>(uintptr_t(256));
    probe.scratch_bytes = ~size_t(0);
    const int nseg = split_segments<float>(probe);
    if (nseg > 1) *bytes = 3 * sizeof(float) * (size_t)a.batch * nseg * a.dim * a.dstate;
    return MB200_OK;
}

extern "C" int mb200_scan_status(int device, int *status)
{
    using namespace mb200;
    if (!status) return fail(MB200_ERR_BAD_ARG, "scan_status: status is NULL");
    if (int rc = enter_device(device)) return rc;
    cudaError_t e = cudaMemcpyFromSymbol(status, g_scan_status, sizeof(int));
    int bwd = 0;
    if (e == cudaSuccess) e = scan_bwd_status(&bwd);
    if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "scan_status: %s", cudaGetErrorString(e));
    if (*status == 0) *status = bwd;
    return MB200_OK;
}

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
