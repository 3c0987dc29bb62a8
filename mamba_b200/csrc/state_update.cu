// Single-token decode state update for sm_100a.
//
// The operator streams the recurrent state once (read + write in place); everything else is a
// few hundred bytes per (batch, head).  The fast kernel therefore gives every state row to a
// group of LPR lanes that each own one 16-byte packet of the row, keeps four rows per group in
// flight before touching any of them, and holds B, C, dt and exp(A dt) of the (batch, head) in
// registers for the whole CTA.  A general kernel (one warp per row, scalar strided accesses)
// serves layouts the packet path cannot: odd dstate, strided or unaligned state, any dtype mix.
#include "common.cuh"

namespace mb200 {

namespace {

constexpr int kThreads = 64;         // many small CTAs hide the per-(batch, head) set-up latency best
constexpr int kRowsInFlight = 4;     // state rows a lane group loads before it touches any of them
constexpr int kMinRowTile = 64;      // state rows per CTA at least (amortises the B / C / dt set-up)

// out rows of a padding entry (state_batch_indices < 0) are defined to be zero.
__device__ void zero_rows(const mb200_ssu_args &a, int b, int h, int p0, int rows)
{
    for (int r = threadIdx.x; r < rows; r += blockDim.x)
        store_any(a.out, a.x_dtype, (int64_t)b * a.out_stride[0] + (int64_t)h * a.out_stride[1] + (int64_t)(p0 + r) * a.out_stride[2], 0.f);
}

template <typename StateT, int LPR, int NC, bool TIED>
__global__ void __launch_bounds__(kThreads) ssu_packet_kernel(const mb200_ssu_args a, const int row_tile)
{
    constexpr int VEC = 16 / sizeof(StateT);
    constexpr int GROUPS = kThreads / LPR;
    const int b = blockIdx.y, h = blockIdx.z;
    const int p0 = blockIdx.x * row_tile;
    const int rows = min(row_tile, a.dim - p0);
    const int lir = threadIdx.x % LPR;   // lane within the row group
    const int group = threadIdx.x / LPR;

    int64_t sb = b;
    if (a.state_batch_indices) {
        const int idx = a.state_batch_indices[b];
        if (idx < 0) {
            zero_rows(a, b, h, p0, rows);
            return;
        }
        sb = idx;
    }
    StateT *state = static_cast<StateT *>(a.state) + sb * a.state_stride[0] + (int64_t)h * a.state_stride[1];
    const int g = h / (a.nheads / a.ngroups);
    const int64_t xo = (int64_t)b * a.x_stride[0] + (int64_t)h * a.x_stride[1];
    const int64_t dto = (int64_t)b * a.dt_stride[0] + (int64_t)h * a.dt_stride[1];
    const int64_t zo = (int64_t)b * a.z_stride[0] + (int64_t)h * a.z_stride[1];
    const int64_t oo = (int64_t)b * a.out_stride[0] + (int64_t)h * a.out_stride[1];

    // The state rows are the only real traffic: put the first round of packets in flight before
    // the (latency-bound) per-(batch, head) set-up below.
    Vec16<StateT> pk[kRowsInFlight][NC];
    auto load_round = [&](int r0) {
#pragma unroll
        for (int u = 0; u < kRowsInFlight; ++u) {
            const int r = r0 + u * GROUPS;
            if (r < rows) {
                StateT *row = state + (int64_t)(p0 + r) * a.state_stride[2];
#pragma unroll
                for (int c = 0; c < NC; ++c) pk[u][c].load(row + (c * LPR + lir) * VEC);
            }
        }
    };
    load_round(group);

    float Bv[NC][VEC], Cv[NC][VEC];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const int n = (c * LPR + lir) * VEC + i;
            Bv[c][i] = load_any(a.B, a.bc_dtype, (int64_t)b * a.B_stride[0] + (int64_t)g * a.B_stride[1] + (int64_t)n * a.B_stride[2]);
            Cv[c][i] = load_any(a.C, a.bc_dtype, (int64_t)b * a.C_stride[0] + (int64_t)g * a.C_stride[1] + (int64_t)n * a.C_stride[2]);
        }

    float dt_tied = 0.f, dA_tied = 0.f;
    if (TIED) {
        dt_tied = load_any(a.dt, a.dt_dtype, dto);
        if (a.dt_bias) dt_tied += a.dt_bias[(int64_t)h * a.dt_bias_stride[0]];
        if (a.dt_softplus) dt_tied = softplus20(dt_tied);
        dA_tied = expf(a.A[(int64_t)h * a.A_stride[0]] * dt_tied);
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int i = 0; i < VEC; ++i) Bv[c][i] *= dt_tied;   // B dt, shared by every row
    }

    // every thread runs the same number of rounds (the shuffles below need whole warps)
    for (int base = 0; base < rows; base += GROUPS * kRowsInFlight) {
        const int r0 = base + group;
        if (base > 0) load_round(r0);
#pragma unroll
        for (int u = 0; u < kRowsInFlight; ++u) {
            const int r = r0 + u * GROUPS;
            const bool live = r < rows;
            const int p = p0 + (live ? r : 0);
            float y = 0.f, xv = 0.f;
            if (live) {
                xv = load_any(a.x, a.x_dtype, xo + (int64_t)p * a.x_stride[2]);
                float dtv = dt_tied;
                if (!TIED) {
                    dtv = load_any(a.dt, a.dt_dtype, dto + (int64_t)p * a.dt_stride[2]);
                    if (a.dt_bias) dtv += a.dt_bias[(int64_t)h * a.dt_bias_stride[0] + (int64_t)p * a.dt_bias_stride[1]];
                    if (a.dt_softplus) dtv = softplus20(dtv);
                }
                StateT *row = state + (int64_t)p * a.state_stride[2];
                const float *Arow = a.A + (int64_t)h * a.A_stride[0] + (int64_t)p * a.A_stride[1];
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    float s[VEC];
                    pk[u][c].unpack(s);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        float dA, dBx;
                        if (TIED) {
                            dA = dA_tied;
                            dBx = Bv[c][i] * xv;
                        } else {
                            const int n = (c * LPR + lir) * VEC + i;
                            dA = __expf(Arow[(int64_t)n * a.A_stride[2]] * dtv);
                            dBx = Bv[c][i] * dtv * xv;
                        }
                        s[i] = fmaf(s[i], dA, dBx);
                        y = fmaf(s[i], Cv[c][i], y);
                    }
                    pk[u][c].pack(s);
                    pk[u][c].store(row + (c * LPR + lir) * VEC);
                }
            }
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
            if (live && lir == 0) {
                if (a.D) y = fmaf(xv, a.D[(int64_t)h * a.D_stride[0] + (int64_t)p * a.D_stride[1]], y);
                if (a.z) y *= silu(load_any(a.z, a.x_dtype, zo + (int64_t)p * a.z_stride[2]));
                store_any(a.out, a.x_dtype, oo + (int64_t)p * a.out_stride[2], y);
            }
        }
    }
}

// One warp per state row, every access scalar and fully strided.
__global__ void __launch_bounds__(128) ssu_general_kernel(const mb200_ssu_args a)
{
    const int b = blockIdx.y, h = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = blockIdx.x * 4 + warp;
    if (p >= a.dim) return;
    const int64_t oi = (int64_t)b * a.out_stride[0] + (int64_t)h * a.out_stride[1] + (int64_t)p * a.out_stride[2];
    int64_t sb = b;
    if (a.state_batch_indices) {
        const int idx = a.state_batch_indices[b];
        if (idx < 0) {
            if (lane == 0) store_any(a.out, a.x_dtype, oi, 0.f);
            return;
        }
        sb = idx;
    }
    const int g = h / (a.nheads / a.ngroups);
    const float xv = load_any(a.x, a.x_dtype, (int64_t)b * a.x_stride[0] + (int64_t)h * a.x_stride[1] + (int64_t)p * a.x_stride[2]);
    float dtv = load_any(a.dt, a.dt_dtype, (int64_t)b * a.dt_stride[0] + (int64_t)h * a.dt_stride[1] + (int64_t)p * a.dt_stride[2]);
    if (a.dt_bias) dtv += a.dt_bias[(int64_t)h * a.dt_bias_stride[0] + (int64_t)p * a.dt_bias_stride[1]];
    if (a.dt_softplus) dtv = softplus20(dtv);
    const int64_t so = sb * a.state_stride[0] + (int64_t)h * a.state_stride[1] + (int64_t)p * a.state_stride[2];
    const float *Arow = a.A + (int64_t)h * a.A_stride[0] + (int64_t)p * a.A_stride[1];
    float y = 0.f;
    for (int n = lane; n < a.dstate; n += 32) {
        const float Bn = load_any(a.B, a.bc_dtype, (int64_t)b * a.B_stride[0] + (int64_t)g * a.B_stride[1] + (int64_t)n * a.B_stride[2]);
        const float Cn = load_any(a.C, a.bc_dtype, (int64_t)b * a.C_stride[0] + (int64_t)g * a.C_stride[1] + (int64_t)n * a.C_stride[2]);
        float s = load_any(a.state, a.state_dtype, so + (int64_t)n * a.state_stride[3]);
        s = fmaf(s, expf(Arow[(int64_t)n * a.A_stride[2]] * dtv), Bn * dtv * xv);
        store_any(a.state, a.state_dtype, so + (int64_t)n * a.state_stride[3], s);
        y = fmaf(s, Cn, y);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
    if (lane == 0) {
        if (a.D) y = fmaf(xv, a.D[(int64_t)h * a.D_stride[0] + (int64_t)p * a.D_stride[1]], y);
        if (a.z) y *= silu(load_any(a.z, a.x_dtype, (int64_t)b * a.z_stride[0] + (int64_t)h * a.z_stride[1] + (int64_t)p * a.z_stride[2]));
        store_any(a.out, a.x_dtype, oi, y);
    }
}

template <typename StateT, int LPR, int NC>
int launch_packet(const mb200_ssu_args &a, bool tied, cudaStream_t stream)
{
    constexpr int GROUPS = kThreads / LPR;
    int row_tile = GROUPS * kRowsInFlight;
    if (row_tile < kMinRowTile) row_tile = kMinRowTile;
    if (row_tile > a.dim) row_tile = a.dim;
    dim3 grid((a.dim + row_tile - 1) / row_tile, a.batch, a.nheads);
    if (tied)
        ssu_packet_kernel<StateT, LPR, NC, true><<<grid, kThreads, 0, stream>>>(a, row_tile);
    else
        ssu_packet_kernel<StateT, LPR, NC, false><<<grid, kThreads, 0, stream>>>(a, row_tile);
    return MB200_OK;
}

template <typename StateT>
bool try_packet(const mb200_ssu_args &a, bool tied, cudaStream_t stream)
{
    constexpr int VEC = 16 / sizeof(StateT);
    if (a.dstate % VEC) return false;
    const int packets = a.dstate / VEC;
    switch (packets) {
    case 2: launch_packet<StateT, 2, 1>(a, tied, stream); return true;
    case 4: launch_packet<StateT, 4, 1>(a, tied, stream); return true;
    case 8: launch_packet<StateT, 8, 1>(a, tied, stream); return true;
    case 16: launch_packet<StateT, 16, 1>(a, tied, stream); return true;
    case 32: launch_packet<StateT, 32, 1>(a, tied, stream); return true;
    case 64: launch_packet<StateT, 32, 2>(a, tied, stream); return true;
    default: return false;
    }
}

bool valid_dtype(int d) { return d == MB200_F32 || d == MB200_F16 || d == MB200_BF16; }

}  // namespace
}  // namespace mb200

extern "C" int mb200_selective_state_update(const mb200_ssu_args *args, void *stream_)
{
    using namespace mb200;
    if (!args) return fail(MB200_ERR_BAD_ARG, "selective_state_update: args is NULL");
    const mb200_ssu_args &a = *args;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    MB200_CHECK_ARG(a.batch >= 0 && a.nheads > 0 && a.dim > 0 && a.dstate > 0 && a.ngroups > 0,
                    "selective_state_update: sizes must be positive (batch %d nheads %d dim %d dstate %d ngroups %d)",
                    a.batch, a.nheads, a.dim, a.dstate, a.ngroups);
    MB200_CHECK_ARG(a.nheads % a.ngroups == 0, "nheads must be divisible by ngroups");
    MB200_CHECK_ARG(valid_dtype(a.state_dtype) && valid_dtype(a.x_dtype) && valid_dtype(a.dt_dtype) && valid_dtype(a.bc_dtype),
                    "selective_state_update: unknown dtype code");
    MB200_CHECK_ARG(a.batch <= 65535 && a.nheads <= 65535, "selective_state_update: batch and nheads must be <= 65535");
    if (a.batch == 0) return MB200_OK;   // nothing to do; empty tensors carry NULL pointers
    MB200_CHECK_ARG(a.state && a.x && a.dt && a.A && a.B && a.C && a.out, "selective_state_update: a required tensor is NULL");
    if (int rc = enter_device(a.device)) return rc;

    const bool tied = a.A_stride[1] == 0 && a.A_stride[2] == 0 && a.dt_stride[2] == 0 &&
                      (!a.dt_bias || a.dt_bias_stride[1] == 0);
    const int vec = 16 / dtype_size(a.state_dtype);
    const bool packet_ok = a.state_stride[3] == 1 && a.state_stride[2] % vec == 0 && a.state_stride[1] % vec == 0 &&
                           a.state_stride[0] % vec == 0 && (reinterpret_cast<uintptr_t>(a.state) & 15) == 0;
    bool done = false;
    if (packet_ok) {
        if (a.state_dtype == MB200_F32) done = try_packet<float>(a, tied, stream);
        else if (a.state_dtype == MB200_BF16) done = try_packet<__nv_bfloat16>(a, tied, stream);
        else done = try_packet<__half>(a, tied, stream);
    }
    if (!done) {
        dim3 grid((a.dim + 3) / 4, a.batch, a.nheads);
        ssu_general_kernel<<<grid, 128, 0, stream>>>(a);
    }
    MB200_CHECK_LAUNCH("selective_state_update");
    return MB200_OK;
}
