// Mamba-1 selective scan, backward (the gradient of selective_scan_fwd with respect to every input).
//
// The reference walks one channel per CTA with the time steps spread over its threads, a forward and a reverse
// block scan per state, and adds every element of dB, dC to global memory atomically
// (csrc/selective_scan/selective_scan_bwd_kernel.cuh).  Here a lane owns a channel and walks time sequentially,
// as the forward does: the two warps of a CTA hold eight states each of the same 32 channels as packed fp32 pairs.
//
//   adjoint:  g_t = C_t dy_t + a_{t+1} g_{t+1}          (a_t = exp(dt_t A), dy_t = dout_t silu(z_t) or dout_t)
//   du_t = D dy_t + dt_t sum_n g_t B_t                   d(dt_t) = sum_n g_t (A a_t h_{t-1} + B_t u_t)
//   dA = sum_t g_t dt_t a_t h_{t-1}                      dB_t = sum_d g_t dt_t u_t        dC_t = sum_d dy_t h_t
//   with a_t h_{t-1} = h_t - dt_t u_t B_t, so only h_t has to be known when the walk comes back to step t.
//
// Two launches per pass over 16 states.  The first walks forward and stores the state before every block of eight
// steps (channel-contiguous, 8 bytes per element and 16 states).  The second walks the blocks from the last to the
// first: eight steps forward from the stored state with the eight h_t kept in registers, then the same eight steps
// backward.  The sums over the channels of a group (dB, dC) are formed inside the warp -- each lane leaves its 16
// values of a step in shared memory, the warp reads them back transposed, a pair of lanes adds up one value -- and
// leave as one vector atomic per four steps, 1/32 of the reference's atomic traffic.  The sums over the states
// (du, d(dt), y for dz) cross the two warps through shared memory.  dstate > 16 repeats both launches per 16 states
// and carries fp32 partial sums of du, ddelta, dz between the passes.
#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "tc_sm100.cuh"
#include "tensor_map.cuh"

namespace mb200 {
namespace {

constexpr int kNS = 16;           // states per pass
constexpr int kBlk = 8;           // steps per block = spacing of the stored states
constexpr int kRedStride = 36;    // row stride (words) of the transposition buffer: 16-byte aligned rows, no bank conflicts
constexpr float kLn2 = 0.6931471805599453f;

// Bounded waits on tile copies record a code here when they run out (0 = never); read through mb200_scan_status.
__device__ int g_scan_bwd_status;
constexpr int kStBwdTile = 41;

// u, delta, dout, z as (seqlen, dim, batch) tensors, fetched as tiles of 8 steps x 32 channels
struct BwdMaps { CUtensorMap u, delta, dout, z, du, ddelta, dz; };

struct BwdPlan {
    int n0;                 // first state of this pass
    int pass, npass;
    int nblk;               // blocks of kBlk steps
    int tiles_per_group;    // CTAs per group (32 channels each, the last one possibly ragged)
    int io_vec, bc_vec;     // rows of the (batch, dim, seqlen) tensors / of B and C may be read in packets
    int tma_out;            // du, ddelta, dz leave as tiles (16-bit outputs, whole tiles of 32 channels per group)
    float *ckpt;            // [batch][nblk][kNS][dim]: state before each block
    float *acc;             // [3][batch][dim][seqlen] fp32: du, ddelta, dz summed over the earlier passes (npass > 1)
};

// CNT consecutive elements of a row, kept as loaded (raw words) so that a prefetch costs few registers.
template <typename T, int CNT> struct Raw {
    static constexpr int W = CNT * (int)sizeof(T) / 4;
    uint32_t w[W];
    __device__ __forceinline__ void load(const T *row, int t0, int L, bool vec)
    {
        if (vec && t0 + CNT <= L) {
            if constexpr (W == 2) {
                const uint2 v = *reinterpret_cast<const uint2 *>(row + t0);
                w[0] = v.x; w[1] = v.y;
            } else {
#pragma unroll
                for (int c = 0; c < W / 4; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(row + t0 + c * (16 / (int)sizeof(T)));
                    w[4 * c] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
                }
            }
        } else {
            T *e = reinterpret_cast<T *>(w);
#pragma unroll
            for (int i = 0; i < CNT; ++i) e[i] = t0 + i < L ? row[t0 + i] : from_float<T>(0.f);
        }
    }
    __device__ __forceinline__ float get(int i) const { return to_float(reinterpret_cast<const T *>(w)[i]); }
};

// softplus with the identity above 20 and its derivative (the logistic function, 1 above 20), sharing one exponential
__device__ __forceinline__ void softplus_and_slope(float x, float &sp, float &slope)
{
    const float t = ex2(-fabsf(x) * kLog2e);          // exp(-|x|) in (0, 1]
    const float r = __fdividef(1.f, 1.f + t);
    const float s = __fdividef(t, 2.f + t), s2 = s * s;
    float p = fmaf(s2, 1.f / 13.f, 1.f / 11.f);
    p = fmaf(p, s2, 1.f / 9.f);
    p = fmaf(p, s2, 1.f / 7.f);
    p = fmaf(p, s2, 1.f / 5.f);
    p = fmaf(p, s2, 1.f / 3.f);
    p = fmaf(p, s2, 1.f);
    sp = fmaf(2.f * s, p, fmaxf(x, 0.f));             // max(x, 0) + log1p(t), log1p(t) = 2 atanh(t / (2 + t))
    slope = x >= 0.f ? r : t * r;
    if (x > 20.f) { sp = x; slope = 1.f; }
}

struct Where {
    int b, g, dbeg, dend, d, lane, w;
    bool active;
};
__device__ __forceinline__ Where where(const BwdPlan &pl, int dim, int ngroups)
{
    Where q;
    q.lane = threadIdx.x & 31;
    q.w = threadIdx.x >> 5;
    q.b = blockIdx.y;
    const int per_group = dim / ngroups;
    q.g = blockIdx.x / pl.tiles_per_group;
    q.dbeg = q.g * per_group + (blockIdx.x % pl.tiles_per_group) * 32;
    q.dend = min(q.dbeg + 32, (q.g + 1) * per_group);
    q.active = q.dbeg + q.lane < q.dend;
    q.d = q.active ? q.dbeg + q.lane : q.dend - 1;     // idle lanes read a valid channel and contribute zeros
    return q;
}

// B (lanes 0-15) and C (lanes 16-31) rows of the pass's 16 states for one block of steps
template <typename T, bool BV, bool CV>
__device__ __forceinline__ const T *bc_row(const mb200_scan_bwd_args &a, const BwdPlan &pl, const Where &q, bool &on)
{
    const bool isC = q.lane >= 16;
    const int n = pl.n0 + (q.lane & 15);
    on = n < a.dstate && (isC ? CV : BV);
    if (!on) return nullptr;
    const int64_t *st = isC ? a.C_stride : a.B_stride;
    return static_cast<const T *>(isC ? a.C : a.B) + (int64_t)q.b * st[0] + (int64_t)q.g * st[1] + (int64_t)n * st[2];
}

// ---------------------------------------------------------------------------------------------- stored states
// Walks forward and stores the state before every block but the first (which is zero).
template <typename T, bool BV, bool TMA>
__global__ void __launch_bounds__(64, 9) scan_bwd_states_kernel(const mb200_scan_bwd_args a, const BwdPlan pl, const __grid_constant__ BwdMaps maps)
{
    constexpr int kTileBytes = 32 * kBlk * (int)sizeof(T);
    __shared__ __align__(128) uint8_t s_tile[TMA ? 2 : 1][TMA ? kTileBytes : 16];   // u, delta: [channel][step]
    __shared__ uint64_t s_full;
    __shared__ int s_dead;
    __shared__ float s_dl[kBlk][32], s_dlu[kBlk][32];
    __shared__ __align__(16) float s_B[kBlk][kNS];
    const Where q = where(pl, a.dim, a.ngroups);
    const int lane = q.lane, w = q.w, L = a.seqlen, N = a.dstate;
    const T *urow = static_cast<const T *>(a.u) + (int64_t)q.b * a.u_stride[0] + (int64_t)q.d * a.u_stride[1];
    const T *drow = static_cast<const T *>(a.delta) + (int64_t)q.b * a.delta_stride[0] + (int64_t)q.d * a.delta_stride[1];
    const float bias = a.delta_bias ? a.delta_bias[q.d] : 0.f;
    bool bc_on = false;
    const T *brow = nullptr;
    if (w == 0) {
        brow = bc_row<T, BV, false>(a, pl, q, bc_on);
        bc_on = bc_on && lane < 16;
    }
    uint64_t A2[4], Bc[4], h[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float av[2], bv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int n = pl.n0 + 8 * w + 2 * j + e;
            const bool valid = n < N && q.active;
            av[e] = valid ? a.A[(int64_t)q.d * a.A_stride[0] + (int64_t)n * a.A_stride[1]] * kLog2e : 0.f;
            bv[e] = (!BV && valid) ? static_cast<const float *>(a.B)[(int64_t)q.d * a.B_stride[0] + (int64_t)n * a.B_stride[1]] : 0.f;
        }
        A2[j] = pack2(av[0], av[1]);
        Bc[j] = pack2(bv[0], bv[1]);
        h[j] = pack2(0.f, 0.f);
    }
    Raw<T, 4> ru, rd;
    Raw<T, 8> rb;
    auto request_tiles = [&](int k) {     // one thread; the tiles of block k-1 have been read by everybody
        tc::mbar_expect_tx(&s_full, 2 * kTileBytes);
        tc::tma_load_3d(s_tile[0], &maps.u, &s_full, k * kBlk, q.dbeg, q.b);
        tc::tma_load_3d(s_tile[1], &maps.delta, &s_full, k * kBlk, q.dbeg, q.b);
    };
    if (TMA) {
        if (threadIdx.x == 0) {
            tc::mbar_init(&s_full, 1);
            tc::mbar_fence_init();
            s_dead = 0;
        }
        __syncthreads();
        if (threadIdx.x == 0) request_tiles(0);
    } else {
        ru.load(urow, 4 * w, L, pl.io_vec);
        rd.load(drow, 4 * w, L, pl.io_vec);
    }
    if (bc_on) rb.load(brow, 0, L, pl.bc_vec);
    for (int k = 0; k + 1 < pl.nblk; ++k) {
        const int t0 = k * kBlk;
        if (TMA) {       // my four steps of my row of each tile
            if (!s_dead && !tc::mbar_wait(&s_full, k & 1, &g_scan_bwd_status, kStBwdTile)) s_dead = 1;
            auto take = [&](int which, Raw<T, 4> &r) {
                const uint8_t *src = s_tile[which] + (lane * kBlk + 4 * w) * (int)sizeof(T);
                if constexpr (sizeof(T) == 4) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(src);
                    r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w;
                } else {
                    const uint2 v = *reinterpret_cast<const uint2 *>(src);
                    r.w[0] = v.x; r.w[1] = v.y;
                }
            };
            take(0, ru);
            take(1, rd);
        }
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
            const int i = 4 * w + i4;
            float dl = rd.get(i4) + bias, slope;
            if (a.delta_softplus) softplus_and_slope(dl, dl, slope);
            if (t0 + i >= L || !q.active) dl = 0.f;
            s_dl[i][lane] = dl;
            s_dlu[i][lane] = dl * ru.get(i4);
        }
        if (BV && w == 0 && lane < 16) {
#pragma unroll
            for (int i = 0; i < kBlk; ++i) s_B[i][lane] = bc_on ? rb.get(i) : 0.f;
        }
        if (!TMA) {
            ru.load(urow, t0 + kBlk + 4 * w, L, pl.io_vec);
            rd.load(drow, t0 + kBlk + 4 * w, L, pl.io_vec);
        }
        if (bc_on) rb.load(brow, t0 + kBlk, L, pl.bc_vec);
        __syncthreads();
        if (TMA && k + 2 < pl.nblk && threadIdx.x == 0 && !s_dead) request_tiles(k + 1);    // everybody has read the tiles of block k
#pragma unroll
        for (int i = 0; i < kBlk; ++i) {
            const float dl = s_dl[i][lane], dlu = s_dlu[i][lane];
            const uint64_t dl2 = pack2(dl, dl), dlu2 = pack2(dlu, dlu);
            uint64_t Bp[4];
            if (BV) {
                const ulonglong2 b01 = *reinterpret_cast<const ulonglong2 *>(&s_B[i][8 * w]);
                const ulonglong2 b23 = *reinterpret_cast<const ulonglong2 *>(&s_B[i][8 * w + 4]);
                Bp[0] = b01.x; Bp[1] = b01.y; Bp[2] = b23.x; Bp[3] = b23.y;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) Bp[j] = Bc[j];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float x0, x1;
                unpack2(mul2(dl2, A2[j]), x0, x1);
                h[j] = fma2(pack2(ex2(x0), ex2(x1)), h[j], mul2(dlu2, Bp[j]));
            }
        }
        if (q.active) {
            float *dst = pl.ckpt + (((int64_t)q.b * pl.nblk + (k + 1)) * kNS + 8 * w) * a.dim + q.d;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float lo, hi;
                unpack2(h[j], lo, hi);
                dst[(int64_t)(2 * j) * a.dim] = lo;
                dst[(int64_t)(2 * j + 1) * a.dim] = hi;
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------- backward walk
// Registers decide how many CTAs an SM holds, and with equal-length CTAs anything short of the whole grid resident
// costs a second round: nine CTAs per SM hold all 1280 channel tiles of an (8, 5120) call at once.  To stay under
// that limit only four of a block's eight h_t are kept at a time: the block is walked forward to its middle, its
// second half forward (kept) and backward, then its first half again from the stored state, forward (kept) and
// backward -- half a forward walk more instead of 32 more registers.
// TMA: the four row tensors arrive as tiles through the copy engine (one request per block from one thread, no
// row-strided loads, no prefetch registers); otherwise every lane reads its own row.
template <typename T, bool BV, bool CV, bool TMA>
__global__ void __launch_bounds__(64, 9) scan_bwd_kernel(const mb200_scan_bwd_args a, const BwdPlan pl, const __grid_constant__ BwdMaps maps)
{
    constexpr int kTileBytes = 32 * kBlk * (int)sizeof(T);
    constexpr bool TMA_OUT = TMA && sizeof(T) == 2;     // fp32 tiles would cost a CTA per SM
    __shared__ __align__(128) uint8_t s_tile[TMA ? 4 : 1][TMA ? kTileBytes : 16];   // u, delta, dout, z: [channel][step]
    __shared__ __align__(128) uint8_t s_out[TMA_OUT ? 3 : 1][TMA_OUT ? kTileBytes : 16];   // du, ddelta, dz
    __shared__ uint64_t s_full;
    __shared__ int s_dead;
    __shared__ float s_dl[kBlk][32], s_dlu[kBlk][32], s_dy[kBlk][32];
    __shared__ float s_u[kBlk][32], s_slope[kBlk][32], s_dzf[kBlk][32];   // of a step, for the warp that finishes it
    __shared__ float s_h0[2][8][32];                               // per warp: the state before the block
    __shared__ __align__(16) float s_BC[kBlk][2 * kNS];            // [step][B of 16 states, C of 16 states]
    __shared__ float s_part[2][3][kBlk][32];                       // per warp: sum g B, sum g (a h) A log2e, sum C h
    __shared__ __align__(16) float s_red[2][16 * kRedStride];      // per warp: 16 values of one step, by lane
    const Where q = where(pl, a.dim, a.ngroups);
    const int lane = q.lane, w = q.w, L = a.seqlen, N = a.dstate;
    const bool has_z = a.z != nullptr;
    const bool first = pl.pass == 0, last = pl.pass == pl.npass - 1;
    const T *urow = static_cast<const T *>(a.u) + (int64_t)q.b * a.u_stride[0] + (int64_t)q.d * a.u_stride[1];
    const T *drow = static_cast<const T *>(a.delta) + (int64_t)q.b * a.delta_stride[0] + (int64_t)q.d * a.delta_stride[1];
    const T *grow = static_cast<const T *>(a.dout) + (int64_t)q.b * a.dout_stride[0] + (int64_t)q.d * a.dout_stride[1];
    const T *zrow = has_z ? static_cast<const T *>(a.z) + (int64_t)q.b * a.z_stride[0] + (int64_t)q.d * a.z_stride[1] : nullptr;
    const float bias = a.delta_bias ? a.delta_bias[q.d] : 0.f;
    const float Dd = (a.D && first) ? a.D[q.d] : 0.f;
    bool bc_on = false;
    const T *bcrow = nullptr;
    if (w == 0) bcrow = bc_row<T, BV, CV>(a, pl, q, bc_on);

    uint64_t A2[4], Bc[4], Cc[4], dA2[4], dBc[4], dCc[4], gc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float av[2], bv[2], cv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int n = pl.n0 + 8 * w + 2 * j + e;
            const bool valid = n < N && q.active;
            av[e] = valid ? a.A[(int64_t)q.d * a.A_stride[0] + (int64_t)n * a.A_stride[1]] * kLog2e : 0.f;
            bv[e] = (!BV && valid) ? static_cast<const float *>(a.B)[(int64_t)q.d * a.B_stride[0] + (int64_t)n * a.B_stride[1]] : 0.f;
            cv[e] = (!CV && valid) ? static_cast<const float *>(a.C)[(int64_t)q.d * a.C_stride[0] + (int64_t)n * a.C_stride[1]] : 0.f;
        }
        A2[j] = pack2(av[0], av[1]);
        Bc[j] = pack2(bv[0], bv[1]);
        Cc[j] = pack2(cv[0], cv[1]);
        dA2[j] = dBc[j] = dCc[j] = gc[j] = pack2(0.f, 0.f);
    }
    float dD_acc = 0.f, dbias_acc = 0.f;

    Raw<T, 4> ru, rd, rg, rz;
    Raw<T, 8> rbc;
    float hck[8];
    auto request_tiles = [&](int k) {     // one thread; the tiles of block k+1 have been read by everybody
        tc::mbar_expect_tx(&s_full, (has_z ? 4 : 3) * kTileBytes);
        tc::tma_load_3d(s_tile[0], &maps.u, &s_full, k * kBlk, q.dbeg, q.b);
        tc::tma_load_3d(s_tile[1], &maps.delta, &s_full, k * kBlk, q.dbeg, q.b);
        tc::tma_load_3d(s_tile[2], &maps.dout, &s_full, k * kBlk, q.dbeg, q.b);
        if (has_z) tc::tma_load_3d(s_tile[3], &maps.z, &s_full, k * kBlk, q.dbeg, q.b);
    };
    auto send_out = [&](int k) {          // one thread; the output tiles of block k are complete
        tc::tma_store_3d(&maps.du, s_out[0], k * kBlk, q.dbeg, q.b);
        tc::tma_store_3d(&maps.ddelta, s_out[1], k * kBlk, q.dbeg, q.b);
        if (has_z) tc::tma_store_3d(&maps.dz, s_out[2], k * kBlk, q.dbeg, q.b);
        tc::tma_store_commit();
    };
    auto fetch = [&](int k) {        // what block k needs from memory through this lane
        const int t = k * kBlk + 4 * w;
        if (!TMA) {
            ru.load(urow, t, L, pl.io_vec);
            rd.load(drow, t, L, pl.io_vec);
            rg.load(grow, t, L, pl.io_vec);
            if (has_z) rz.load(zrow, t, L, pl.io_vec);
        }
        if (bc_on) rbc.load(bcrow, k * kBlk, L, pl.bc_vec);
        if (k > 0 && q.active) {
            const float *src = pl.ckpt + (((int64_t)q.b * pl.nblk + k) * kNS + 8 * w) * a.dim + q.d;
#pragma unroll
            for (int j = 0; j < 8; ++j) hck[j] = src[(int64_t)j * a.dim];
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) hck[j] = 0.f;
        }
    };
    if (TMA) {
        if (threadIdx.x == 0) {
            tc::mbar_init(&s_full, 1);
            tc::mbar_fence_init();
            s_dead = 0;
        }
        __syncthreads();
        if (threadIdx.x == 0) request_tiles(pl.nblk - 1);
    }
    fetch(pl.nblk - 1);

    for (int k = pl.nblk - 1; k >= 0; --k) {
        const int t0 = k * kBlk;
        if (TMA) {       // my four steps of my row of each tile
            // a wait that ran out has recorded its code; s_dead (set by whichever thread saw it, read unsynchronised:
            // every thread of the CTA waits on the same barrier and gives up on its own) only keeps the CTA from
            // spending another time limit per block on its way out
            if (!s_dead && !tc::mbar_wait(&s_full, (pl.nblk - 1 - k) & 1, &g_scan_bwd_status, kStBwdTile)) s_dead = 1;
            auto take = [&](int which, Raw<T, 4> &r) {
                const uint8_t *src = s_tile[which] + (lane * kBlk + 4 * w) * (int)sizeof(T);
                if constexpr (sizeof(T) == 4) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(src);
                    r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w;
                } else {
                    const uint2 v = *reinterpret_cast<const uint2 *>(src);
                    r.w[0] = v.x; r.w[1] = v.y;
                }
            };
            take(0, ru);
            take(1, rd);
            take(2, rg);
            if (has_z) take(3, rz);
        }
        // ---- scalars of my four steps, B and C of the block
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
            const int i = 4 * w + i4;
            const bool in = t0 + i < L && q.active;
            float dl = rd.get(i4) + bias, slope = 1.f;
            if (a.delta_softplus) softplus_and_slope(dl, dl, slope);
            float uu = ru.get(i4), go = rg.get(i4), dy = go, dzf = 0.f;
            if (has_z) {
                const float zz = rz.get(i4);
                const float sg = __fdividef(1.f, 1.f + ex2(-zz * kLog2e));
                dy = go * zz * sg;
                dzf = go * sg * fmaf(zz, 1.f - sg, 1.f);
            }
            if (!in) { dl = 0.f; uu = 0.f; dy = 0.f; dzf = 0.f; slope = 0.f; }
            s_dl[i][lane] = dl;
            s_dlu[i][lane] = dl * uu;
            s_dy[i][lane] = dy;
            s_u[i][lane] = uu;
            s_slope[i][lane] = slope;
            s_dzf[i][lane] = dzf;
        }
        if ((BV || CV) && w == 0) {
#pragma unroll
            for (int i = 0; i < kBlk; ++i) s_BC[i][lane] = bc_on ? rbc.get(i) : 0.f;
        }
        uint64_t h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            h[j] = pack2(hck[2 * j], hck[2 * j + 1]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s_h0[w][j][lane] = hck[j];
        if (k > 0) fetch(k - 1);
        __syncthreads();
        if (TMA && k > 0 && threadIdx.x == 0 && !s_dead) request_tiles(k - 1);     // everybody has read the tiles of block k
        const bool out_tiles = TMA_OUT && pl.tma_out && last;
        if (out_tiles && k + 1 < pl.nblk && threadIdx.x == 0) send_out(k + 1);      // block k+1's outputs are complete in s_out

        auto load_B = [&](int i, uint64_t (&Bp)[4]) {
            if (BV) {
                const ulonglong2 b01 = *reinterpret_cast<const ulonglong2 *>(&s_BC[i][8 * w]);
                const ulonglong2 b23 = *reinterpret_cast<const ulonglong2 *>(&s_BC[i][8 * w + 4]);
                Bp[0] = b01.x; Bp[1] = b01.y; Bp[2] = b23.x; Bp[3] = b23.y;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) Bp[j] = Bc[j];
            }
        };
        auto load_C = [&](int i, uint64_t (&Cp)[4]) {
            if (CV) {
                const ulonglong2 c01 = *reinterpret_cast<const ulonglong2 *>(&s_BC[i][kNS + 8 * w]);
                const ulonglong2 c23 = *reinterpret_cast<const ulonglong2 *>(&s_BC[i][kNS + 8 * w + 4]);
                Cp[0] = c01.x; Cp[1] = c01.y; Cp[2] = c23.x; Cp[3] = c23.y;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) Cp[j] = Cc[j];
            }
        };
        auto step_forward = [&](int i) {
            const float dl = s_dl[i][lane], dlu = s_dlu[i][lane];
            const uint64_t dl2 = pack2(dl, dl), dlu2 = pack2(dlu, dlu);
            uint64_t Bp[4];
            load_B(i, Bp);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float x0, x1;
                unpack2(mul2(dl2, A2[j]), x0, x1);
                h[j] = fma2(pack2(ex2(x0), ex2(x1)), h[j], mul2(dlu2, Bp[j]));
            }
        };

        // ---- forward to the middle of the block; then per half: forward with every h_t kept, and backward
#pragma unroll
        for (int i = 0; i < 4; ++i) step_forward(i);
        float res[kBlk];     // (variable B, C) lane pair v = lane / 2: sum over the channels of value v, per step
#pragma unroll
        for (int half = 1; half >= 0; --half) {
            if (half == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = pack2(s_h0[w][2 * j][lane], s_h0[w][2 * j + 1][lane]);
            }
            uint64_t hs[4][4];
#pragma unroll
            for (int i4 = 0; i4 < 4; ++i4) {
                const int i = 4 * half + i4;
                step_forward(i);
#pragma unroll
                for (int j = 0; j < 4; ++j) hs[i4][j] = h[j];
                if (has_z) {      // y_t, which only dz needs
                    uint64_t Cp[4];
                    load_C(i, Cp);
                    uint64_t y2 = mul2(h[0], Cp[0]);
#pragma unroll
                    for (int j = 1; j < 4; ++j) y2 = fma2(h[j], Cp[j], y2);
                    float y0, y1;
                    unpack2(y2, y0, y1);
                    s_part[w][2][i][lane] = y0 + y1;
                }
            }
#pragma unroll
            for (int i4 = 3; i4 >= 0; --i4) {
                const int i = 4 * half + i4;
                const float dl = s_dl[i][lane], dlu = s_dlu[i][lane], dy = s_dy[i][lane];
                const uint64_t dl2 = pack2(dl, dl), dlu2 = pack2(dlu, dlu), dy2 = pack2(dy, dy);
                uint64_t Bp[4], Cp[4];
                load_B(i, Bp);
                load_C(i, Cp);
                uint64_t s1 = pack2(0.f, 0.f), s2 = pack2(0.f, 0.f);
                float *red = s_red[w];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint64_t g = fma2(Cp[j], dy2, gc[j]);                 // g_t
                    const uint64_t ah = sub2(hs[i4][j], mul2(dlu2, Bp[j]));     // a_t h_{t-1}
                    const uint64_t gah = mul2(g, ah);
                    dA2[j] = fma2(gah, dl2, dA2[j]);
                    s1 = fma2(g, Bp[j], s1);
                    s2 = fma2(gah, A2[j], s2);
                    const uint64_t db = mul2(g, dlu2), dc = mul2(hs[i4][j], dy2);
                    if (BV) {
                        float lo, hi;
                        unpack2(db, lo, hi);
                        red[(2 * j) * kRedStride + lane] = lo;
                        red[(2 * j + 1) * kRedStride + lane] = hi;
                    } else {
                        dBc[j] = add2(dBc[j], db);
                    }
                    if (CV) {
                        float lo, hi;
                        unpack2(dc, lo, hi);
                        red[(8 + 2 * j) * kRedStride + lane] = lo;
                        red[(8 + 2 * j + 1) * kRedStride + lane] = hi;
                    } else {
                        dCc[j] = add2(dCc[j], dc);
                    }
                    float x0, x1;
                    unpack2(mul2(dl2, A2[j]), x0, x1);
                    gc[j] = mul2(pack2(ex2(x0), ex2(x1)), g);                   // a_t g_t, what step t-1 receives
                }
                {
                    float lo, hi;
                    unpack2(s1, lo, hi);
                    s_part[w][0][i][lane] = lo + hi;
                    unpack2(s2, lo, hi);
                    s_part[w][1][i][lane] = lo + hi;
                }
                if (BV || CV) {
                    // lane pair v reads back row v (16 lanes each); with only one of B, C input-dependent the other half of
                    // the rows was never written, and what the pairs 8-15 (or 0-7) add up there is dropped below
                    __syncwarp();
                    const float4 *src = reinterpret_cast<const float4 *>(red + (lane >> 1) * kRedStride + (lane & 1) * 16);
                    const float4 p0 = src[0], p1 = src[1], p2 = src[2], p3 = src[3];
                    float s = ((p0.x + p0.y) + (p0.z + p0.w)) + ((p1.x + p1.y) + (p1.z + p1.w)) + ((p2.x + p2.y) + (p2.z + p2.w)) +
                              ((p3.x + p3.y) + (p3.z + p3.w));
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    res[i] = s;
                    __syncwarp();
                }
            }
        }
        if (BV || CV) {
            // lane pair v: tensor v / 8 (dB, dC), state n0 + 8 w + v % 8; the even lane adds steps 0-3, the odd one 4-7
            const int v = lane >> 1, half = lane & 1;
            const bool isC = v >= 8;
            const int n = pl.n0 + 8 * w + (v & 7);
            if (n < N && (isC ? CV : BV)) {
                float *dst = (isC ? a.dC : a.dB) + (((int64_t)q.b * a.ngroups + q.g) * N + n) * L + t0 + 4 * half;
                const float r0 = half ? res[4] : res[0], r1 = half ? res[5] : res[1], r2 = half ? res[6] : res[2],
                            r3 = half ? res[7] : res[3];
                if ((L & 3) == 0 && t0 + 4 * half + 4 <= L) {
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(r0), "f"(r1), "f"(r2), "f"(r3) : "memory");
                } else {
                    const float r[4] = {r0, r1, r2, r3};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (t0 + 4 * half + e < L) atomicAdd(dst + e, r[e]);
                }
            }
        }
        if (out_tiles && threadIdx.x == 0) tc::tma_store_wait_read();     // the tiles of block k+1 have left shared memory
        __syncthreads();

        // ---- sums over the 16 states, my four steps
        float o_du[4], o_dd[4], o_dz[4];
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
            const int i = 4 * w + i4;
            const float S1 = s_part[0][0][i][lane] + s_part[1][0][i][lane];
            const float S2 = s_part[0][1][i][lane] + s_part[1][1][i][lane];
            const float uu = s_u[i][lane], dy = s_dy[i][lane];
            o_du[i4] = fmaf(s_dl[i][lane], S1, Dd * dy);
            o_dd[i4] = fmaf(kLn2, S2, uu * S1) * s_slope[i][lane];
            o_dz[i4] = 0.f;
            if (has_z) o_dz[i4] = fmaf(Dd, uu, s_part[0][2][i][lane] + s_part[1][2][i][lane]) * s_dzf[i][lane];
            dD_acc = fmaf(uu, dy, dD_acc);
            dbias_acc += o_dd[i4];
        }
        if (q.active) {
            const int t = t0 + 4 * w;
            if (pl.npass > 1) {     // partial sums of the passes over other states
                float *acc = pl.acc + ((int64_t)q.b * a.dim + q.d) * L + t;
                const int64_t plane = (int64_t)a.batch * a.dim * L;
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    if (t + i4 >= L) break;
                    if (!first) {
                        o_du[i4] += acc[i4];
                        o_dd[i4] += acc[plane + i4];
                        if (has_z) o_dz[i4] += acc[2 * plane + i4];
                    }
                    if (!last) {
                        acc[i4] = o_du[i4];
                        acc[plane + i4] = o_dd[i4];
                        if (has_z) acc[2 * plane + i4] = o_dz[i4];
                    }
                }
            }
            if (out_tiles) {
                if constexpr (TMA_OUT) {
                    auto park = [&](int which, const float (&v)[4]) {
                        uint2 o;
                        T *e = reinterpret_cast<T *>(&o);
#pragma unroll
                        for (int i4 = 0; i4 < 4; ++i4) e[i4] = from_float<T>(v[i4]);
                        *reinterpret_cast<uint2 *>(s_out[which] + (lane * kBlk + 4 * w) * (int)sizeof(T)) = o;
                    };
                    park(0, o_du);
                    park(1, o_dd);
                    if (has_z) park(2, o_dz);
                    tc::fence_proxy_async();
                }
            } else if (last) {
                auto put = [&](void *base, const int64_t *st, const float (&v)[4]) {
                    T *row = static_cast<T *>(base) + (int64_t)q.b * st[0] + (int64_t)q.d * st[1] + t;
                    if (pl.io_vec && t + 4 <= L) {
                        if constexpr (sizeof(T) == 4) {
                            *reinterpret_cast<float4 *>(row) = make_float4(v[0], v[1], v[2], v[3]);
                        } else {
                            uint2 o;
                            T *e = reinterpret_cast<T *>(&o);
#pragma unroll
                            for (int i4 = 0; i4 < 4; ++i4) e[i4] = from_float<T>(v[i4]);
                            *reinterpret_cast<uint2 *>(row) = o;
                        }
                    } else {
#pragma unroll
                        for (int i4 = 0; i4 < 4; ++i4)
                            if (t + i4 < L) row[i4] = from_float<T>(v[i4]);
                    }
                };
                put(a.du, a.du_stride, o_du);
                put(a.ddelta, a.ddelta_stride, o_dd);
                if (has_z) put(a.dz, a.dz_stride, o_dz);
            }
        }
        // The next block's scalar phase rewrites the rows of s_dl .. s_dzf that this warp itself has just read (each warp
        // prepares and finishes the same four steps), but the other warp's forward walk of that block must not start
        // before they are complete and this block's reads are done: the barrier after the scalar phase orders both.
        // s_part is rewritten only after that barrier, which the reads above precede.
    }

    if (TMA_OUT && pl.tma_out && last) {      // the outputs of block 0
        __syncthreads();
        if (threadIdx.x == 0) {
            send_out(0);
            tc::tma_store_wait_read();
        }
    }
    if (q.active) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v[2], vb[2], vc[2];
            unpack2(dA2[j], v[0], v[1]);
            unpack2(dBc[j], vb[0], vb[1]);
            unpack2(dCc[j], vc[0], vc[1]);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = pl.n0 + 8 * w + 2 * j + e;
                if (n >= N) continue;
                atomicAdd(a.dA + (int64_t)q.d * N + n, v[e]);
                if (!BV) atomicAdd(a.dB + (int64_t)q.d * N + n, vb[e]);
                if (!CV) atomicAdd(a.dC + (int64_t)q.d * N + n, vc[e]);
            }
        }
        if (a.dD && first) atomicAdd(a.dD + q.d, dD_acc);
        if (a.ddelta_bias) atomicAdd(a.ddelta_bias + q.d, dbias_acc);
    }
}

bool aligned_to(const void *p, size_t n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; }

// Scratch per batch row: the stored states and, above 16 states, the partial sums carried between the passes.  Batch
// rows are independent, so a large batch is walked in slices that re-use one scratch of at most kScratchCap bytes (one
// row if a single row needs more).
constexpr size_t kScratchCap = size_t(1) << 30;
size_t ckpt_floats_per_row(const mb200_scan_bwd_args &a) { return (((size_t)a.seqlen + kBlk - 1) / kBlk) * kNS * a.dim; }
size_t acc_floats_per_row(const mb200_scan_bwd_args &a) { return a.dstate > kNS ? 3 * (size_t)a.dim * a.seqlen : 0; }
size_t row_bytes(const mb200_scan_bwd_args &a) { return sizeof(float) * (ckpt_floats_per_row(a) + acc_floats_per_row(a)); }
int rows_under_cap(const mb200_scan_bwd_args &a)
{
    const size_t per_row = row_bytes(a);
    if (per_row == 0) return a.batch;
    const size_t rows = kScratchCap / per_row;
    return (int)(rows < 1 ? 1 : rows > (size_t)a.batch ? (size_t)a.batch : rows);
}

template <typename T, bool BV, bool CV>
void launch_pass(const mb200_scan_bwd_args &a, const BwdPlan &pl, dim3 grid, cudaStream_t stream, const BwdMaps *maps)
{
    if (maps) {
        if (pl.nblk > 1) scan_bwd_states_kernel<T, BV, true><<<grid, 64, 0, stream>>>(a, pl, *maps);
        scan_bwd_kernel<T, BV, CV, true><<<grid, 64, 0, stream>>>(a, pl, *maps);
    } else {
        static const BwdMaps none = {};
        if (pl.nblk > 1) scan_bwd_states_kernel<T, BV, false><<<grid, 64, 0, stream>>>(a, pl, none);
        scan_bwd_kernel<T, BV, CV, false><<<grid, 64, 0, stream>>>(a, pl, none);
    }
}

// Tensor maps of the four row tensors of this slice; false when a tensor cannot be described (the lanes then read
// their rows themselves).
template <typename T>
bool encode_rows(const mb200_scan_bwd_args &a, BwdMaps &m)
{
    if (!encode_fn()) return false;
    const int dtype = sizeof(T) == 4 ? MB200_F32 : (std::is_same<T, __half>::value ? MB200_F16 : MB200_BF16);
    auto one = [&](CUtensorMap *map, const void *p, const int64_t *st) {
        const uint64_t dims[3] = {(uint64_t)a.seqlen, (uint64_t)a.dim, (uint64_t)a.batch};
        const uint64_t sb[2] = {(uint64_t)st[1] * sizeof(T), (uint64_t)st[0] * sizeof(T)};
        const uint32_t box[3] = {(uint32_t)kBlk, 32u, 1u};
        return st[0] > 0 && st[1] > 0 && encode_tiled(map, dtype, p, 3, dims, sb, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    };
    bool ok = one(&m.u, a.u, a.u_stride) && one(&m.delta, a.delta, a.delta_stride) && one(&m.dout, a.dout, a.dout_stride) &&
              one(&m.du, a.du, a.du_stride) && one(&m.ddelta, a.ddelta, a.ddelta_stride);
    if (a.z) ok = ok && one(&m.z, a.z, a.z_stride) && one(&m.dz, a.dz, a.dz_stride);
    else { m.z = m.u; m.dz = m.du; }
    return ok;
}

template <typename T>
int launch_slice(const mb200_scan_bwd_args &a, cudaStream_t stream);

// Walks the batch in slices of as many rows as the lent scratch holds.
template <typename T>
int launch_bwd(const mb200_scan_bwd_args &a, cudaStream_t stream)
{
    const size_t per_row = row_bytes(a);
    const int rows = per_row ? (int)std::min<size_t>((size_t)a.batch, a.scratch_bytes / per_row) : a.batch;
    for (int b0 = 0; b0 < a.batch; b0 += rows) {
        mb200_scan_bwd_args s = a;
        s.batch = std::min(rows, a.batch - b0);
        auto adv = [&](const void *p, int64_t stride) { return p ? static_cast<const void *>(static_cast<const char *>(p) + (int64_t)b0 * stride * (int64_t)sizeof(T)) : p; };
        s.u = adv(a.u, a.u_stride[0]);
        s.delta = adv(a.delta, a.delta_stride[0]);
        s.z = adv(a.z, a.z_stride[0]);
        s.dout = adv(a.dout, a.dout_stride[0]);
        s.du = const_cast<void *>(adv(a.du, a.du_stride[0]));
        s.ddelta = const_cast<void *>(adv(a.ddelta, a.ddelta_stride[0]));
        s.dz = const_cast<void *>(adv(a.dz, a.dz_stride[0]));
        const int64_t vrow = (int64_t)a.ngroups * a.dstate * a.seqlen;      // dB, dC: fp32, contiguous
        if (a.B_variable) {
            s.B = adv(a.B, a.B_stride[0]);
            s.dB = a.dB + (int64_t)b0 * vrow;
        }
        if (a.C_variable) {
            s.C = adv(a.C, a.C_stride[0]);
            s.dC = a.dC + (int64_t)b0 * vrow;
        }
        if (int rc = launch_slice<T>(s, stream)) return rc;
    }
    return MB200_OK;
}

template <typename T>
int launch_slice(const mb200_scan_bwd_args &a, cudaStream_t stream)
{
    constexpr int VEC = 16 / sizeof(T);
    auto rows_ok = [&](const void *p, const int64_t *s) { return aligned_to(p, 16) && s[0] % VEC == 0 && s[1] % VEC == 0; };
    BwdPlan pl;
    pl.io_vec = rows_ok(a.u, a.u_stride) && rows_ok(a.delta, a.delta_stride) && rows_ok(a.dout, a.dout_stride) &&
                rows_ok(a.du, a.du_stride) && rows_ok(a.ddelta, a.ddelta_stride) &&
                (!a.z || (rows_ok(a.z, a.z_stride) && rows_ok(a.dz, a.dz_stride)));
    pl.bc_vec = 1;
    if (a.B_variable) pl.bc_vec = pl.bc_vec && aligned_to(a.B, 16) && a.B_stride[0] % VEC == 0 && a.B_stride[1] % VEC == 0 && a.B_stride[2] % VEC == 0;
    if (a.C_variable) pl.bc_vec = pl.bc_vec && aligned_to(a.C, 16) && a.C_stride[0] % VEC == 0 && a.C_stride[1] % VEC == 0 && a.C_stride[2] % VEC == 0;
    pl.nblk = (a.seqlen + kBlk - 1) / kBlk;
    const int per_group = a.dim / a.ngroups;
    pl.tiles_per_group = (per_group + 31) / 32;
    // Output tiles need whole channel tiles (a ragged tile's idle lanes would store into the next group's rows) and rows
    // that end on a 16-byte boundary: a tile store clips the innermost dimension in 16-byte units, not in elements, so
    // a row of a wider buffer that ends inside such a unit would have the bytes after its end overwritten.
    pl.tma_out = per_group % 32 == 0 && ((size_t)a.seqlen * sizeof(T)) % 16 == 0;
    pl.npass = (a.dstate + kNS - 1) / kNS;
    pl.ckpt = static_cast<float *>(a.scratch);
    pl.acc = pl.ckpt + (size_t)a.batch * ckpt_floats_per_row(a);
    dim3 grid(a.ngroups * pl.tiles_per_group, a.batch);
    BwdMaps maps;
    const BwdMaps *use = (pl.io_vec && encode_rows<T>(a, maps)) ? &maps : nullptr;
    for (int p = 0; p < pl.npass; ++p) {
        pl.pass = p;
        pl.n0 = p * kNS;
        if (a.B_variable && a.C_variable) launch_pass<T, true, true>(a, pl, grid, stream, use);
        else if (a.B_variable) launch_pass<T, true, false>(a, pl, grid, stream, use);
        else if (a.C_variable) launch_pass<T, false, true>(a, pl, grid, stream, use);
        else launch_pass<T, false, false>(a, pl, grid, stream, use);
    }
    return MB200_OK;
}

int check_bwd(const mb200_scan_bwd_args &a)
{
    MB200_CHECK_ARG(a.batch >= 0 && a.dim > 0 && a.seqlen >= 0 && a.dstate > 0 && a.ngroups > 0,
                    "selective_scan_bwd: bad sizes (batch %d dim %d seqlen %d dstate %d ngroups %d)", a.batch, a.dim, a.seqlen,
                    a.dstate, a.ngroups);
    MB200_CHECK_ARG(a.dstate <= 256, "selective_scan only supports state dimension <= 256");
    MB200_CHECK_ARG(a.dim % a.ngroups == 0, "selective_scan_bwd: dim must be divisible by ngroups");
    MB200_CHECK_ARG(a.io_dtype == MB200_F32 || a.io_dtype == MB200_F16 || a.io_dtype == MB200_BF16,
                    "selective_scan_bwd: unknown io_dtype %d", a.io_dtype);
    MB200_CHECK_ARG(a.batch <= 65535, "selective_scan_bwd: batch must be <= 65535");
    return MB200_OK;
}

}  // namespace

cudaError_t scan_bwd_status(int *status) { return cudaMemcpyFromSymbol(status, g_scan_bwd_status, sizeof(int)); }

}  // namespace mb200

extern "C" int mb200_scan_bwd_scratch_bytes(const mb200_scan_bwd_args *args, size_t *bytes)
{
    using namespace mb200;
    if (!args || !bytes) return fail(MB200_ERR_BAD_ARG, "scan_bwd_scratch_bytes: NULL argument");
    *bytes = 0;
    if (int rc = check_bwd(*args)) return rc;
    *bytes = (size_t)rows_under_cap(*args) * row_bytes(*args) + 16;
    return MB200_OK;
}

extern "C" int mb200_selective_scan_bwd(const mb200_scan_bwd_args *args, void *stream_)
{
    using namespace mb200;
    if (!args) return fail(MB200_ERR_BAD_ARG, "selective_scan_bwd: args is NULL");
    const mb200_scan_bwd_args &a = *args;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_bwd(a)) return rc;
    MB200_CHECK_ARG(a.A && a.dA, "selective_scan_bwd: A or dA is NULL");
    MB200_CHECK_ARG(!a.D == !a.dD, "selective_scan_bwd: dD goes with D");
    MB200_CHECK_ARG(!a.delta_bias == !a.ddelta_bias, "selective_scan_bwd: ddelta_bias goes with delta_bias");
    MB200_CHECK_ARG(aligned_to(a.dB, 16) && aligned_to(a.dC, 16), "selective_scan_bwd: dB and dC must be 16-byte aligned");
    if (int rc = enter_device(a.device)) return rc;
    // the accumulators start from zero (selective_scan.cpp:460-465 allocates them with zeros); empty tensors carry NULL
    const size_t wn = sizeof(float) * (size_t)a.dim * a.dstate;
    const size_t vn = sizeof(float) * (size_t)a.batch * a.ngroups * a.dstate * a.seqlen;
    const size_t bn = a.B_variable ? vn : wn, cn = a.C_variable ? vn : wn;
    cudaError_t e = cudaMemsetAsync(a.dA, 0, wn, stream);
    if (e == cudaSuccess && a.dB && bn) e = cudaMemsetAsync(a.dB, 0, bn, stream);
    if (e == cudaSuccess && a.dC && cn) e = cudaMemsetAsync(a.dC, 0, cn, stream);
    if (e == cudaSuccess && a.dD) e = cudaMemsetAsync(a.dD, 0, sizeof(float) * a.dim, stream);
    if (e == cudaSuccess && a.ddelta_bias) e = cudaMemsetAsync(a.ddelta_bias, 0, sizeof(float) * a.dim, stream);
    if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "selective_scan_bwd: memset: %s", cudaGetErrorString(e));
    if (a.batch == 0 || a.seqlen == 0) return MB200_OK;
    MB200_CHECK_ARG(a.u && a.delta && a.B && a.C && a.dout && a.du && a.ddelta && a.dB && a.dC,
                    "selective_scan_bwd: a required tensor is NULL");
    MB200_CHECK_ARG(!a.z || a.dz, "selective_scan_bwd: dz is required with z");
    const size_t need = row_bytes(a);      // at least one batch row at a time
    MB200_CHECK_ARG(a.scratch && a.scratch_bytes >= need && aligned_to(a.scratch, 16),
                    "selective_scan_bwd: scratch of at least %zu bytes, 16-byte aligned, is required (got %zu)", need, a.scratch_bytes);
    int rc;
    if (a.io_dtype == MB200_F32) rc = launch_bwd<float>(a, stream);
    else if (a.io_dtype == MB200_BF16) rc = launch_bwd<__nv_bfloat16>(a, stream);
    else rc = launch_bwd<__half>(a, stream);
    if (rc) return rc;
    MB200_CHECK_LAUNCH("selective_scan_bwd");
    return MB200_OK;
}
