// Mamba-2 SSD chunked forward for sm_100a: stage kernels that work for every shape and dtype.
//
// Stages (each one launch, all on the caller's stream, handing fp32 intermediates through the
// caller's scratch buffer):
//   1. chunk_cumsum   dt <- clamp(softplus(dt + bias)), dA_cum <- cumsum_Q(dt A)
//   2. chunk_state    S_c[p,n] = sum_k x[k,p] B[k,n] exp(min(dA_last - dA_k, 0)) dt_k
//   3. state_passing  H_{c+1} = exp(dA_last_c) H_c + S_c, slot c rewritten with H_c
//   4. chunk_cb       CB[m,k] = C_m . B_k   (lower block triangle)
//   5. chunk_scan     y_m = exp(dA_m) C_m.H_c + sum_{k<=m} CB[m,k] exp(min(dA_m - dA_k,0)) dt_k x_k + D x_m,
//                     then y_m * silu(z_m)
// The contractions here run on the fp32 FMA pipes through a 64x64 shared-memory tile loop, which
// keeps fp32 inputs exact; the bf16/fp16 tensor-core tiles for the benchmark shapes live in
// ssd_tc.cu and replace stages 2, 4 and 5 when the shape qualifies.
#include <algorithm>

#include "ssd_common.cuh"

namespace mb200 {
namespace {

constexpr int kT = 256;       // threads per CTA in the tile kernels
constexpr int kKT = 32;       // reduction step
constexpr int kLd = 68;       // padded leading dimension of the staged tiles (keeps float4 alignment)

// acc[4][4] += A[64 x K] * B[K x 64] for the thread's 4x4 patch (rows ty*4.., cols tx*4..).
// fa(k, i) / fb(k, j) return the (bounds-checked) operand elements; *_KFAST says the source is
// contiguous along k, which only changes which thread fetches which element.
template <bool A_KFAST, bool B_KFAST, class FA, class FB>
__device__ __forceinline__ void tile_gemm(float (&acc)[4][4], int K, FA fa, FB fb, float *As, float *Bs)
{
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    for (int k0 = 0; k0 < K; k0 += kKT) {
        __syncthreads();
        for (int e = threadIdx.x; e < kKT * 64; e += kT) {
            int kk, i;
            if (A_KFAST) { i = e / kKT; kk = e % kKT; } else { kk = e / 64; i = e % 64; }
            As[kk * kLd + i] = (k0 + kk < K) ? fa(k0 + kk, i) : 0.f;
        }
        for (int e = threadIdx.x; e < kKT * 64; e += kT) {
            int kk, j;
            if (B_KFAST) { j = e / kKT; kk = e % kKT; } else { kk = e / 64; j = e % 64; }
            Bs[kk * kLd + j] = (k0 + kk < K) ? fb(k0 + kk, j) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < kKT; ++kk) {
            const float4 av = *reinterpret_cast<const float4 *>(As + kk * kLd + ty * 4);
            const float4 bv = *reinterpret_cast<const float4 *>(Bs + kk * kLd + tx * 4);
            const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
    }
}

// Sequence id of position t of batch row b (packed sequences), or 0 when no ids were given.
__device__ __forceinline__ int seq_at(const mb200_ssd_args &a, int b, int t)
{
    return a.seq_idx ? a.seq_idx[(int64_t)b * a.seqlen + t] : 0;
}

// ---- stage 1 ------------------------------------------------------------------------------------
// One CTA per (chunk, batch, 32 heads): coalesced read of dt over heads, transposed in shared
// memory, then a warp scan along the chunk per head.
template <typename TD>
__global__ void __launch_bounds__(256) ssd_cumsum_kernel(const mb200_ssd_args a, float *dt_out, float *dA_out, int nchunks, uint8_t *seq_start,
                                                         uint8_t *seq_carry)
{
    extern __shared__ float sm[];   // Q x 33
    const int Q = a.chunk_size;
    const int c = blockIdx.x, b = blockIdx.y, h0 = blockIdx.z * 32;
    const int t0 = c * Q;
    // a thread keeps one head (lane) and walks the steps 32 at a time: the loads are issued back to back so
    // that their latencies overlap instead of adding up
    const int hh = threadIdx.x & 31, h = h0 + hh;
    const bool h_ok = h < a.nheads;
    const float bias = (h_ok && a.dt_bias) ? a.dt_bias[h] : 0.f;
    const TD *src = static_cast<const TD *>(a.dt) + (int64_t)b * a.dt_stride[0] + (int64_t)h * a.dt_stride[2];
    constexpr int NB = 32;          // loads in flight per thread: a whole chunk of 256 steps in one round trip
    for (int k0 = threadIdx.x >> 5; k0 < Q; k0 += 8 * NB) {
        TD raw[NB];
#pragma unroll
        for (int u = 0; u < NB; ++u) {
            const int k = k0 + 8 * u;
            raw[u] = (h_ok && k < Q && t0 + k < a.seqlen) ? src[(int64_t)(t0 + k) * a.dt_stride[1]] : from_float<TD>(0.f);
        }
#pragma unroll
        for (int u = 0; u < NB; ++u) {
            const int k = k0 + 8 * u;
            if (k < Q) {
                float v = 0.f;
                if (h_ok && t0 + k < a.seqlen) {
                    v = to_float(raw[u]) + bias;
                    if (a.dt_softplus) v = fast_softplus20(v);
                    v = fminf(fmaxf(v, a.dt_min), a.dt_max);
                }
                sm[k * 33 + hh] = v;
            }
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int hh = warp; hh < 32; hh += 8) {
        const int h = h0 + hh;
        if (h >= a.nheads) break;
        const float A = a.A[h];
        float carry = 0.f;
        const int64_t o = (((int64_t)b * a.nheads + h) * nchunks + c) * Q;
        for (int k0 = 0; k0 < Q; k0 += 32) {
            const int k = k0 + lane;
            const float dtv = k < Q ? sm[k * 33 + hh] : 0.f;
            float v = dtv * A;
#pragma unroll
            for (int o2 = 1; o2 < 32; o2 <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, v, o2);
                if (lane >= o2) v += up;
            }
            v += carry;
            if (k < Q) {
                dt_out[o + k] = dtv;
                dA_out[o + k] = v;
            }
            carry = __shfl_sync(0xffffffffu, v, 31);
        }
    }
    // Packed sequences on the tensor-core path (chunk of 256 = one position per thread): where, inside the chunk, the
    // sequence of every position starts, and whether the chunk's first position continues the previous chunk's last
    // sequence.  The chunk-scan kernel masks with these two instead of comparing ids.
    if (seq_start && blockIdx.z == 0) {
        __syncthreads();            // the transposing buffer is free
        int *wmax = reinterpret_cast<int *>(sm);
        const int32_t *sid = a.seq_idx + (int64_t)b * a.seqlen;
        const int k = threadIdx.x;
        const int me = sid[min(t0 + k, a.seqlen - 1)];
        const int before = k > 0 ? sid[min(t0 + k - 1, a.seqlen - 1)] : me;
        int start = (k > 0 && me != before) ? k : 0;            // a sequence starts here
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) start = max(start, __shfl_up_sync(0xffffffffu, start, o) * (lane >= o ? 1 : 0));
        if (lane == 31) wmax[warp] = start;
        __syncthreads();
        for (int w2 = 0; w2 < warp; ++w2) start = max(start, wmax[w2]);
        seq_start[((int64_t)b * nchunks + c) * Q + k] = (uint8_t)start;
        if (k == 0) seq_carry[(int64_t)b * nchunks + c] = me == (c > 0 ? sid[t0 - 1] : 0) ? 1 : 0;
    }
    // When launched as the programmatic dependent of the C.B^T kernel this grid runs alongside it; it must not be
    // complete before that kernel is, because later launches only wait for this one.  (Returns at once otherwise.)
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- stage 2 ------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kT) ssd_chunk_state_kernel(const mb200_ssd_args a, const float *dtb, const float *dAb,
                                                             float *states, int nchunks)
{
    __shared__ __align__(16) float As[kKT * kLd], Bs[kKT * kLd];
    const int Q = a.chunk_size, P = a.headdim, N = a.dstate;
    const int tilesN = (N + 63) / 64;
    const int p0 = (blockIdx.x / tilesN) * 64, n0 = (blockIdx.x % tilesN) * 64;
    const int b = blockIdx.y / nchunks, c = blockIdx.y % nchunks, h = blockIdx.z;
    const int g = h / (a.nheads / a.ngroups);
    const int t0 = c * Q;
    const int len = min(Q, a.seqlen - t0);
    const float *dtc = dtb + (((int64_t)b * a.nheads + h) * nchunks + c) * Q;
    const float *dAc = dAb + (((int64_t)b * a.nheads + h) * nchunks + c) * Q;
    const float dA_last = dAc[Q - 1];
    const T *x = static_cast<const T *>(a.x) + (int64_t)b * a.x_stride[0] + (int64_t)t0 * a.x_stride[1] + (int64_t)h * a.x_stride[2];
    const T *B = static_cast<const T *>(a.B) + (int64_t)b * a.B_stride[0] + (int64_t)t0 * a.B_stride[1] + (int64_t)g * a.B_stride[2];
    float acc[4][4] = {};
    const int seq_last = seq_at(a, b, t0 + len - 1);    // only steps of the chunk's last sequence reach its end state
    tile_gemm<false, false>(
        acc, len,
        [&](int k, int i) {
            if (p0 + i >= P || (a.seq_idx && seq_at(a, b, t0 + k) != seq_last)) return 0.f;
            return to_float(x[(int64_t)k * a.x_stride[1] + p0 + i]) * (__expf(fminf(dA_last - dAc[k], 0.f)) * dtc[k]);
        },
        [&](int k, int j) { return n0 + j < N ? to_float(B[(int64_t)k * a.B_stride[1] + n0 + j]) : 0.f; }, As, Bs);
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float *S = states + (((int64_t)b * nchunks + c) * a.nheads + h) * (int64_t)P * N;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int p = p0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (p < P && n < N) S[(int64_t)p * N + n] = acc[i][j];
        }
}

// ---- stage 3 ------------------------------------------------------------------------------------
// Elementwise over P*N, serial over chunks.  Slot c of `states` receives the state entering chunk c;
// with `prev16` the entering states go there as 16-bit values (the tensor-core chunk_scan reads them
// by TMA) and the fp32 slots are left alone.  VEC elements per thread and kAhead chunks of loads in
// flight keep enough bytes in the air to stream at HBM speed.
template <int VEC>
__global__ void __launch_bounds__(256) ssd_state_passing_kernel(const mb200_ssd_args a, const float *dAb, float *states,
                                                                int nchunks, bool write_prev, void *prev16)
{
    constexpr int kAhead = 4;
    const int64_t PN = (int64_t)a.headdim * a.dstate;
    const int64_t e = ((int64_t)blockIdx.x * 256 + threadIdx.x) * VEC;
    const int h = blockIdx.y, b = blockIdx.z;
    const int Q = a.chunk_size;
    const float *dA_last = dAb + ((int64_t)b * a.nheads + h) * nchunks * Q + (Q - 1);
    if (e < PN) {
        float run[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) run[i] = a.initial_states ? a.initial_states[((int64_t)b * a.nheads + h) * PN + e + i] : 0.f;
        for (int c0 = 0; c0 < nchunks; c0 += kAhead) {
            float s[kAhead][VEC], dec[kAhead];
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int c = c0 + u;
                if (c < nchunks) {
                    const float *slot = states + (((int64_t)b * nchunks + c) * a.nheads + h) * PN + e;
                    if (VEC == 4) {
                        const float4 v = *reinterpret_cast<const float4 *>(slot);
                        s[u][0] = v.x; s[u][1 % VEC] = v.y; s[u][2 % VEC] = v.z; s[u][3 % VEC] = v.w;
                    } else {
                        s[u][0] = slot[0];
                    }
                    dec[u] = __expf(dA_last[(int64_t)c * Q]);
                    if (a.seq_idx) {   // a new sequence at the end of this chunk: nothing carries over from the previous one
                        const int s_new = seq_at(a, b, min((c + 1) * Q, a.seqlen) - 1);
                        const int s_old = c > 0 ? seq_at(a, b, c * Q - 1) : 0;
                        if (s_new != s_old) dec[u] = 0.f;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kAhead; ++u) {
                const int c = c0 + u;
                if (c < nchunks) {
                    const int64_t o = (((int64_t)b * nchunks + c) * a.nheads + h) * PN + e;
                    if (write_prev) {
#pragma unroll
                        for (int i = 0; i < VEC; ++i) {
                            if (prev16) store_any(prev16, a.io_dtype, o + i, run[i]);
                            else states[o + i] = run[i];
                        }
                    }
#pragma unroll
                    for (int i = 0; i < VEC; ++i) run[i] = fmaf(dec[u], run[i], s[u][i]);
                }
            }
        }
        if (a.final_states) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) a.final_states[((int64_t)b * a.nheads + h) * PN + e + i] = run[i];
        }
    }
    if (a.range_decay && blockIdx.x == 0 && threadIdx.x == 0) {
        float tot = 0.f;
        for (int c = 0; c < nchunks; ++c) tot += dA_last[(int64_t)c * Q];
        a.range_decay[(int64_t)b * a.nheads + h] = __expf(tot);
    }
}

// ---- stage 4 ------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kT) ssd_cb_kernel(const mb200_ssd_args a, float *cb, int nchunks)
{
    __shared__ __align__(16) float As[kKT * kLd], Bs[kKT * kLd];
    const int Q = a.chunk_size, N = a.dstate;
    const int tiles = (Q + 63) / 64;
    const int m0 = (blockIdx.x / tiles) * 64, k0 = (blockIdx.x % tiles) * 64;
    if (k0 > m0) return;   // strictly upper blocks are never read
    const int b = blockIdx.y / nchunks, c = blockIdx.y % nchunks, g = blockIdx.z;
    const int t0 = c * Q;
    const int len = min(Q, a.seqlen - t0);
    const T *C = static_cast<const T *>(a.C) + (int64_t)b * a.C_stride[0] + (int64_t)t0 * a.C_stride[1] + (int64_t)g * a.C_stride[2];
    const T *B = static_cast<const T *>(a.B) + (int64_t)b * a.B_stride[0] + (int64_t)t0 * a.B_stride[1] + (int64_t)g * a.B_stride[2];
    float acc[4][4] = {};
    tile_gemm<true, true>(
        acc, N, [&](int n, int i) { return m0 + i < len ? to_float(C[(int64_t)(m0 + i) * a.C_stride[1] + n]) : 0.f; },
        [&](int n, int j) { return k0 + j < len ? to_float(B[(int64_t)(k0 + j) * a.B_stride[1] + n]) : 0.f; }, As, Bs);
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    float *out = cb + (((int64_t)b * nchunks + c) * a.ngroups + g) * (int64_t)Q * Q;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, k = k0 + tx * 4 + j;
            if (m < Q && k < Q) {
                const bool same = !a.seq_idx || (m < len && k < len && seq_at(a, b, t0 + m) == seq_at(a, b, t0 + k));
                out[(int64_t)m * Q + k] = same ? acc[i][j] : 0.f;
            }
        }
}

// ---- stage 5 ------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kT) ssd_chunk_scan_kernel(const mb200_ssd_args a, const float *dtb, const float *dAb,
                                                            const float *states, const float *cb, int nchunks)
{
    __shared__ __align__(16) float As[kKT * kLd], Bs[kKT * kLd];
    const int Q = a.chunk_size, P = a.headdim, N = a.dstate;
    const int tilesP = (P + 63) / 64;
    const int m0 = (blockIdx.x / tilesP) * 64, p0 = (blockIdx.x % tilesP) * 64;
    const int b = blockIdx.y / nchunks, c = blockIdx.y % nchunks, h = blockIdx.z;
    const int g = h / (a.nheads / a.ngroups);
    const int t0 = c * Q;
    const int len = min(Q, a.seqlen - t0);
    if (m0 >= len) return;
    const float *dtc = dtb + (((int64_t)b * a.nheads + h) * nchunks + c) * Q;
    const float *dAc = dAb + (((int64_t)b * a.nheads + h) * nchunks + c) * Q;
    const T *x = static_cast<const T *>(a.x) + (int64_t)b * a.x_stride[0] + (int64_t)t0 * a.x_stride[1] + (int64_t)h * a.x_stride[2];
    const T *C = static_cast<const T *>(a.C) + (int64_t)b * a.C_stride[0] + (int64_t)t0 * a.C_stride[1] + (int64_t)g * a.C_stride[2];
    const float *prev = states + (((int64_t)b * nchunks + c) * a.nheads + h) * (int64_t)P * N;
    const float *cbc = cb + (((int64_t)b * nchunks + c) * a.ngroups + g) * (int64_t)Q * Q;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;

    float acc[4][4] = {};
    // contribution of the state entering the chunk: exp(dA_m) * C_m . H[p,:]
    tile_gemm<true, true>(
        acc, N, [&](int n, int i) { return m0 + i < len ? to_float(C[(int64_t)(m0 + i) * a.C_stride[1] + n]) : 0.f; },
        [&](int n, int j) { return p0 + j < P ? prev[(int64_t)(p0 + j) * N + n] : 0.f; }, As, Bs);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        float sc = m < len ? __expf(dAc[m]) : 0.f;
        // the entering state belongs to the sequence that ends the previous chunk
        if (a.seq_idx && m < len && seq_at(a, b, t0 + m) != (c > 0 ? seq_at(a, b, t0 - 1) : 0)) sc = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] *= sc;
    }
    // causal intra-chunk part
    const int kend = min(m0 + 64, len);
    tile_gemm<true, false>(
        acc, kend,
        [&](int k, int i) {
            const int m = m0 + i;
            return (m < len && k <= m) ? cbc[(int64_t)m * Q + k] * __expf(fminf(dAc[m] - dAc[k], 0.f)) * dtc[k] : 0.f;
        },
        [&](int k, int j) { return p0 + j < P ? to_float(x[(int64_t)k * a.x_stride[1] + p0 + j]) : 0.f; }, As, Bs);

    const T *z = a.z ? static_cast<const T *>(a.z) + (int64_t)b * a.z_stride[0] + (int64_t)t0 * a.z_stride[1] + (int64_t)h * a.z_stride[2] : nullptr;
    T *out = static_cast<T *>(a.out) + (int64_t)b * a.out_stride[0] + (int64_t)t0 * a.out_stride[1] + (int64_t)h * a.out_stride[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= len) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int p = p0 + tx * 4 + j;
            if (p >= P) continue;
            float y = acc[i][j];
            if (a.D) y = fmaf(to_float(x[(int64_t)m * a.x_stride[1] + p]), a.D_has_hdim ? a.D[(int64_t)h * P + p] : a.D[h], y);
            if (z) y *= silu(to_float(z[(int64_t)m * a.z_stride[1] + p]));
            out[(int64_t)m * a.out_stride[1] + p] = from_float<T>(y);
        }
    }
}

// ---- packed sequences: state after the last token of each one ------------------------------------
// One thread per (p, n) element of one (sequence, head): the contribution of the sequence's steps inside
// the chunk that holds its last token, plus the state entering that chunk if the sequence began earlier.
template <typename T>
__global__ void __launch_bounds__(256) ssd_varlen_state_kernel(const mb200_ssd_args a, const float *dtb, const float *dAb,
                                                               const float *states, int nchunks, const void *prev16, int prev_np)
{
    const int P = a.headdim, N = a.dstate, Q = a.chunk_size;
    const int e = blockIdx.x * 256 + threadIdx.x;
    const int s = blockIdx.y, h = blockIdx.z;
    if (e >= P * N) return;
    const int p = e / N, n = e % N;
    const int g = h / (a.nheads / a.ngroups);
    const int start = a.cu_seqlens[s], end = a.cu_seqlens[s + 1];
    float *dst = a.varlen_states + (((int64_t)s * a.nheads + h) * P + p) * N + n;
    if (end <= start || end > a.seqlen) {
        *dst = 0.f;
        return;
    }
    const int c = (end - 1) / Q;
    const int t0 = c * Q;
    const float *dtc = dtb + ((int64_t)h * nchunks + c) * Q;
    const float *dAc = dAb + ((int64_t)h * nchunks + c) * Q;
    const float dA_end = dAc[end - 1 - t0];
    const T *x = static_cast<const T *>(a.x) + (int64_t)h * a.x_stride[2] + p;
    const T *B = static_cast<const T *>(a.B) + (int64_t)g * a.B_stride[2] + n;
    float acc = 0.f;
    for (int t = max(start, t0); t < end; ++t)
        acc = fmaf(to_float(x[(int64_t)t * a.x_stride[1]]) * (__expf(fminf(dA_end - dAc[t - t0], 0.f)) * dtc[t - t0]),
                   to_float(B[(int64_t)t * a.B_stride[1]]), acc);
    if (start < t0) {
        // the state entering chunk c: fp32 [p][n] from the general stages; on the tensor-core path the 16-bit copy the
        // chunk scan reads, [n][p] when the streaming launch wrote it
        const int64_t slot = (((int64_t)c) * a.nheads + h) * (int64_t)P * N;
        const float entering = prev16 ? load_any(prev16, a.io_dtype, slot + (prev_np ? (int64_t)n * P + p : (int64_t)e)) : states[slot + e];
        acc = fmaf(entering, __expf(dA_end), acc);
    }
    *dst = acc;
}

__global__ void ssd_fill_kernel(float *dst, float v, int64_t n)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = v;
}

__global__ void ssd_fold_kernel(const float *s_in, const float *decay, const float *s_local, float *s_out, int64_t rows,
                                int64_t row)
{
    const int64_t total = rows * row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const float in = s_in ? s_in[i] : 0.f;
        s_out[i] = fmaf(decay[i / row], in, s_local[i]);
    }
}

__global__ void ssd_fold_ranges_kernel(const float *summaries, int64_t record_stride, int first, int last, float *s_out, int64_t rows,
                                       int64_t row)
{
    const int64_t total = rows * row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float s = summaries[(int64_t)first * record_stride + i];
        for (int r = first + 1; r <= last; ++r) {
            const float *rec = summaries + (int64_t)r * record_stride;
            s = fmaf(rec[total + i / row], s, rec[i]);
        }
        s_out[i] = s;
    }
}

template <typename T>
int run_ssd(const mb200_ssd_args &a, const SsdScratch &lay, cudaStream_t stream)
{
    char *base = static_cast<char *>(a.scratch);
    float *dtb = reinterpret_cast<float *>(base + lay.off_dt);
    float *dAb = reinterpret_cast<float *>(base + lay.off_dA);
    float *states = reinterpret_cast<float *>(base + lay.off_states);
    float *cb = reinterpret_cast<float *>(base + lay.off_cb);
    const int nc = lay.nchunks, Q = a.chunk_size;
    const int64_t PN = (int64_t)a.headdim * a.dstate;
    // Path choice.  The LOCAL stages (cumsum, chunk states, recurrence) read x, B and dt; the OUTPUT stages add C,
    // z and out.  A whole-operator call takes the tensor-core path only when both halves can; in a sequence split
    // each half decides from what IT reads, so an OUTPUT call can tell how the earlier LOCAL call ran even though
    // that call never saw C, z or out.
    const bool has_local = (a.phases & MB200_SSD_PHASE_LOCAL) != 0, has_out = (a.phases & MB200_SSD_PHASE_OUTPUT) != 0;
    const bool tc_out = ssd_tc_local_eligible(a) && ssd_tc_output_eligible(a);     // OUTPUT stages on tensor cores
    const bool tc_loc = (has_local && has_out) ? tc_out : ssd_tc_local_eligible(a);  // LOCAL stages on tensor cores
    // C.B^T ahead of the exchange of a sequence split: on tensor cores when x, B and C qualify, which both halves can
    // tell (they are handed the same C); the OUTPUT half uses it only if it is the form its chunk scan reads.
    const bool tc_cb_early = ssd_tc_local_eligible(a) && ssd_tc_cb_eligible(a);
    const bool cb_early = has_local && !has_out && (a.phases & MB200_SSD_PHASE_CB) && a.C;
    const bool cb_ready = !has_local && has_out && (a.phases & MB200_SSD_PHASE_CB_READY) && tc_out == tc_cb_early;
    void *prev16 = tc_out ? static_cast<void *>(base + lay.off_prev16) : nullptr;
    {
        cudaError_t e = cudaMemsetAsync(base + lay.off_status, 0, sizeof(int), stream);
        if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "ssd: status reset: %s", cudaGetErrorString(e));
    }
    // Chunk states + inter-chunk recurrence in one streaming launch.  In a sequence split the LOCAL phase runs it
    // from a zero state (entering states of the range as if nothing came in, range summary), and the OUTPUT phase
    // adds the incoming state's share to those entering states: H_c += prefix_decay_c * S_in.
    const bool fused_states = tc_loc && ssd_tc_stream_eligible(a);
    // The LOCAL half took the streaming launch but this OUTPUT half cannot use its 16-bit entering states: the
    // scratch holds no fp32 chunk states, so they are formed here before the recurrence.
    const bool local_streamed = !has_local && fused_states && !tc_out;
    if (a.phases & MB200_SSD_PHASE_LOCAL) {
        const size_t cs_smem = sizeof(float) * Q * 33;
        if (cs_smem > 48 * 1024) {
            cudaError_t e = ensure_dynamic_smem(reinterpret_cast<const void *>(&ssd_cumsum_kernel<float>), (int)cs_smem, a.device);
            if (e == cudaSuccess) e = ensure_dynamic_smem(reinterpret_cast<const void *>(&ssd_cumsum_kernel<__nv_bfloat16>), (int)cs_smem, a.device);
            if (e == cudaSuccess) e = ensure_dynamic_smem(reinterpret_cast<const void *>(&ssd_cumsum_kernel<__half>), (int)cs_smem, a.device);
            if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "ssd chunk_cumsum: shared memory opt-in: %s", cudaGetErrorString(e));
        }
        // C.B^T needs nothing the other stages produce: when the whole operator runs on the tensor-core path it goes
        // first and the cumsum is launched as its programmatic dependent, so the two small kernels share the GPU.
        const bool cb_first = (tc_out && has_out) || (cb_early && tc_cb_early);
        if (cb_first)
            if (int rc = ssd_tc_cb_and_scan(a, lay, fused_states, stream, 1)) return rc;
        if (cb_early && !tc_cb_early) {
            const int tq = (Q + 63) / 64;
            ssd_cb_kernel<T><<<dim3(tq * tq, a.batch * nc, a.ngroups), kT, 0, stream>>>(a, cb, nc);
            MB200_CHECK_LAUNCH("ssd chunk_cb");
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(nc, a.batch, (a.nheads + 31) / 32);
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = cs_smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = cb_first ? 1 : 0;
        int ncv = nc;
        // the sequence-start table is only read by the tensor-core chunk scan (chunk of 256 positions = one per thread)
        uint8_t *seq_start = (a.seq_idx && tc_out) ? reinterpret_cast<uint8_t *>(base + lay.off_seq_start) : nullptr;
        uint8_t *seq_carry = reinterpret_cast<uint8_t *>(base + lay.off_seq_carry);
        cudaError_t ce;
        if (a.dt_dtype == MB200_F32) ce = cudaLaunchKernelEx(&cfg, ssd_cumsum_kernel<float>, a, dtb, dAb, ncv, seq_start, seq_carry);
        else if (a.dt_dtype == MB200_BF16) ce = cudaLaunchKernelEx(&cfg, ssd_cumsum_kernel<__nv_bfloat16>, a, dtb, dAb, ncv, seq_start, seq_carry);
        else ce = cudaLaunchKernelEx(&cfg, ssd_cumsum_kernel<__half>, a, dtb, dAb, ncv, seq_start, seq_carry);
        if (ce != cudaSuccess) return fail(MB200_ERR_LAUNCH, "ssd chunk_cumsum: %s", cudaGetErrorString(ce));
        MB200_CHECK_LAUNCH("ssd chunk_cumsum");
        if (fused_states) {
            if (int rc = ssd_tc_state_stream(a, lay, stream)) return rc;
        } else if (tc_loc) {
            if (int rc = ssd_tc_chunk_state(a, lay, stream)) return rc;
        } else {
            ssd_chunk_state_kernel<T><<<dim3(((a.headdim + 63) / 64) * ((a.dstate + 63) / 64), a.batch * nc, a.nheads), kT, 0, stream>>>(
                a, dtb, dAb, states, nc);
            MB200_CHECK_LAUNCH("ssd chunk_state");
        }
        if (!fused_states && !(a.phases & MB200_SSD_PHASE_OUTPUT) && (a.final_states || a.range_decay)) {
            // range summary only: fold the local chunk states from a zero state, leave the slots as they are
            mb200_ssd_args z = a;
            z.initial_states = nullptr;
            if (PN % 4 == 0)
                ssd_state_passing_kernel<4><<<dim3((unsigned)((PN / 4 + 255) / 256), a.nheads, a.batch), 256, 0, stream>>>(z, dAb, states, nc, false, nullptr);
            else
                ssd_state_passing_kernel<1><<<dim3((unsigned)((PN + 255) / 256), a.nheads, a.batch), 256, 0, stream>>>(z, dAb, states, nc, false, nullptr);
            MB200_CHECK_LAUNCH("ssd range summary");
        }
    }
    if (a.phases & MB200_SSD_PHASE_OUTPUT) {
        mb200_ssd_args p = a;
        if (!(a.phases & MB200_SSD_PHASE_LOCAL)) p.range_decay = nullptr;
        if (local_streamed)      // x and B qualified for the tensor-core chunk-state kernel (that is why LOCAL streamed)
            if (int rc = ssd_tc_chunk_state(a, lay, stream)) return rc;
        if (fused_states && tc_out) {
            // the entering states and the final state come from the state-stream kernel; in the OUTPUT half of a
            // sequence split the incoming state is added to what the LOCAL half left
            if (!(a.phases & MB200_SSD_PHASE_LOCAL))
                if (int rc = ssd_tc_apply_incoming(a, lay, stream)) return rc;
        } else if (PN % 4 == 0) {
            ssd_state_passing_kernel<4><<<dim3((unsigned)((PN / 4 + 255) / 256), a.nheads, a.batch), 256, 0, stream>>>(p, dAb, states, nc, true, prev16);
        } else {
            ssd_state_passing_kernel<1><<<dim3((unsigned)((PN + 255) / 256), a.nheads, a.batch), 256, 0, stream>>>(p, dAb, states, nc, true, prev16);
        }
        MB200_CHECK_LAUNCH("ssd state_passing");
        if (tc_out) {
            // C.B^T already ran ahead of the cumsum when this call includes the LOCAL phase
            if (int rc = ssd_tc_cb_and_scan(a, lay, fused_states, stream, (has_local || cb_ready) ? 2 : 3)) return rc;
        } else {
            const int tq = (Q + 63) / 64;
            if (!cb_ready) {
                ssd_cb_kernel<T><<<dim3(tq * tq, a.batch * nc, a.ngroups), kT, 0, stream>>>(a, cb, nc);
                MB200_CHECK_LAUNCH("ssd chunk_cb");
            }
            ssd_chunk_scan_kernel<T><<<dim3(tq * ((a.headdim + 63) / 64), a.batch * nc, a.nheads), kT, 0, stream>>>(a, dtb, dAb, states, cb, nc);
            MB200_CHECK_LAUNCH("ssd chunk_scan");
        }
        if (a.cu_seqlens && a.varlen_states && a.num_seqs > 0) {
            ssd_varlen_state_kernel<T><<<dim3((unsigned)((PN + 255) / 256), a.num_seqs, a.nheads), 256, 0, stream>>>(a, dtb, dAb, states, nc, prev16,
                                                                                                                   (fused_states && tc_out) ? 1 : 0);
            MB200_CHECK_LAUNCH("ssd varlen states");
        }
    }
    return MB200_OK;
}

int check_ssd(const mb200_ssd_args &a)
{
    MB200_CHECK_ARG(a.batch >= 0 && a.seqlen >= 0 && a.nheads > 0 && a.headdim > 0 && a.ngroups > 0 && a.dstate > 0 && a.chunk_size > 0,
                    "ssd: bad sizes (batch %d seqlen %d nheads %d headdim %d ngroups %d dstate %d chunk %d)", a.batch, a.seqlen,
                    a.nheads, a.headdim, a.ngroups, a.dstate, a.chunk_size);
    MB200_CHECK_ARG(a.nheads % a.ngroups == 0, "nheads must be divisible by ngroups");
    MB200_CHECK_ARG(a.io_dtype == MB200_F32 || a.io_dtype == MB200_F16 || a.io_dtype == MB200_BF16, "ssd: unknown io_dtype %d", a.io_dtype);
    MB200_CHECK_ARG(a.dt_dtype == MB200_F32 || a.dt_dtype == MB200_F16 || a.dt_dtype == MB200_BF16, "ssd: unknown dt_dtype %d", a.dt_dtype);
    MB200_CHECK_ARG(a.chunk_size <= 1024, "ssd: chunk_size must be <= 1024");
    MB200_CHECK_ARG((a.phases & MB200_SSD_PHASE_ALL) != 0 && (a.phases & ~(MB200_SSD_PHASE_ALL | MB200_SSD_PHASE_CB | MB200_SSD_PHASE_CB_READY)) == 0,
                    "ssd: phases must be a combination of LOCAL and OUTPUT");
    MB200_CHECK_ARG(!(a.phases & MB200_SSD_PHASE_CB) || (a.phases & MB200_SSD_PHASE_ALL) == MB200_SSD_PHASE_LOCAL, "ssd: PHASE_CB goes with a LOCAL-only call");
    MB200_CHECK_ARG(!(a.phases & MB200_SSD_PHASE_CB_READY) || (a.phases & MB200_SSD_PHASE_ALL) == MB200_SSD_PHASE_OUTPUT,
                    "ssd: PHASE_CB_READY goes with an OUTPUT-only call");
    return MB200_OK;
}

}  // namespace
}  // namespace mb200

extern "C" int mb200_ssd_scratch_bytes(const mb200_ssd_args *args, size_t *bytes)
{
    using namespace mb200;
    if (!args || !bytes) return fail(MB200_ERR_BAD_ARG, "ssd_scratch_bytes: NULL argument");
    if (int rc = check_ssd(*args)) return rc;
    *bytes = ssd_scratch_layout(*args).total;
    return MB200_OK;
}

extern "C" int mb200_ssd_chunk_scan_fwd(const mb200_ssd_args *args, void *stream_)
{
    using namespace mb200;
    if (!args) return fail(MB200_ERR_BAD_ARG, "ssd_chunk_scan_fwd: args is NULL");
    const mb200_ssd_args &a = *args;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (int rc = check_ssd(a)) return rc;
    MB200_CHECK_ARG(!(a.phases & MB200_SSD_PHASE_OUTPUT) || a.out || a.seqlen == 0 || a.batch == 0, "ssd: out is NULL");
    MB200_CHECK_ARG(!a.cu_seqlens || a.batch == 1, "passing cu_seqlens to get the varlen states is only supported if batch dimension is 1");
    MB200_CHECK_ARG(!a.cu_seqlens || (a.num_seqs >= 0 && a.num_seqs <= 65535), "ssd: num_seqs must be in [0, 65535]");
    MB200_CHECK_ARG(!(a.seq_idx || a.cu_seqlens) || (a.phases & MB200_SSD_PHASE_ALL) == MB200_SSD_PHASE_ALL, "ssd: packed sequences cannot be combined with a sequence split");
    if (a.batch == 0) return MB200_OK;   // nothing to do; empty tensors carry NULL pointers
    MB200_CHECK_ARG(a.seqlen == 0 || (a.x && a.dt && a.A && a.B && a.C), "ssd: a required tensor is NULL");
    if (int rc = enter_device(a.device)) return rc;
    MB200_CHECK_ARG(a.batch * (int64_t)((a.seqlen + a.chunk_size - 1) / a.chunk_size) <= 65535 && a.nheads <= 65535 && a.batch <= 65535,
                    "ssd: batch*nchunks and nheads must be <= 65535");
    const SsdScratch lay = ssd_scratch_layout(a);
    if (a.seqlen == 0) {
        const size_t n = sizeof(float) * (size_t)a.batch * a.nheads * a.headdim * a.dstate;
        if (a.final_states && (a.phases & MB200_SSD_PHASE_OUTPUT)) {
            cudaError_t e = a.initial_states ? cudaMemcpyAsync(a.final_states, a.initial_states, n, cudaMemcpyDeviceToDevice, stream)
                                             : cudaMemsetAsync(a.final_states, 0, n, stream);
            if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "ssd: final state copy: %s", cudaGetErrorString(e));
        } else if ((a.phases & MB200_SSD_PHASE_ALL) == MB200_SSD_PHASE_LOCAL) {
            // an empty range of a sequence split is summarised by the identity: state 0, decay 1
            if (a.final_states) {
                const cudaError_t e = cudaMemsetAsync(a.final_states, 0, n, stream);
                if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "ssd: empty range state: %s", cudaGetErrorString(e));
            }
            if (a.range_decay) {
                const int64_t rows = (int64_t)a.batch * a.nheads;
                ssd_fill_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, stream>>>(a.range_decay, 1.f, rows);
                MB200_CHECK_LAUNCH("ssd: empty range decay");
            }
        }
        return MB200_OK;
    }
    MB200_CHECK_ARG(a.scratch && a.scratch_bytes >= lay.total, "ssd: scratch too small (%zu < %zu bytes)", a.scratch_bytes, lay.total);
    MB200_CHECK_ARG((reinterpret_cast<uintptr_t>(a.scratch) & 255) == 0, "ssd: scratch must be 256-byte aligned");
    if (a.io_dtype == MB200_F32) return run_ssd<float>(a, lay, stream);
    if (a.io_dtype == MB200_BF16) return run_ssd<__nv_bfloat16>(a, lay, stream);
    return run_ssd<__half>(a, lay, stream);
}

// ---- the variant that allocates nothing ---------------------------------------------------------------
// The intermediates of the SSD stages for callers that cannot allocate: a fixed buffer inside the
// library image.  In host code this name is only a handle for the runtime, not a device address; the
// address each device gave it is fetched once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_ssd_static_scratch[MB200_SSD_STATIC_SCRATCH_BYTES];

extern "C" int mb200_ssd_chunk_scan_fwd_static(const mb200_ssd_args *args, void *stream)
{
    using namespace mb200;
    if (!args) return fail(MB200_ERR_BAD_ARG, "ssd_chunk_scan_fwd_static: args is NULL");
    if (int rc = check_ssd(*args)) return rc;
    const size_t need = ssd_scratch_layout(*args).total;
    if (need > MB200_SSD_STATIC_SCRATCH_BYTES)
        return fail(MB200_ERR_BAD_ARG,
                    "ssd_chunk_scan_fwd_static: this problem needs %zu bytes of intermediates, the built-in buffer holds %u; "
                    "use mb200_ssd_chunk_scan_fwd with caller-owned scratch",
                    need, (unsigned)MB200_SSD_STATIC_SCRATCH_BYTES);
    if (args->batch == 0) return MB200_OK;
    if (int rc = enter_device(args->device)) return rc;
    // one look-up per device, made with that device current (enter_device did that)
    static void *device_address[64] = {nullptr};
    void *ptr = device_address[args->device];
    if (!ptr) {
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_ssd_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(MB200_ERR_LAUNCH, "ssd_chunk_scan_fwd_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        device_address[args->device] = ptr;
    }
    mb200_ssd_args a = *args;
    a.scratch = ptr;
    a.scratch_bytes = MB200_SSD_STATIC_SCRATCH_BYTES;
    return mb200_ssd_chunk_scan_fwd(&a, stream);
}

extern "C" int mb200_ssd_static_status(const mb200_ssd_args *args, int *status)
{
    using namespace mb200;
    if (!args || !status) return fail(MB200_ERR_BAD_ARG, "ssd_static_status: NULL argument");
    if (int rc = check_ssd(*args)) return rc;
    const SsdScratch lay = ssd_scratch_layout(*args);
    if (lay.total > MB200_SSD_STATIC_SCRATCH_BYTES) return fail(MB200_ERR_BAD_ARG, "ssd_static_status: this problem does not fit the built-in buffer");
    if (int rc = enter_device(args->device)) return rc;
    // synchronises with the device: a diagnostic, not part of the hot path
    const cudaError_t e = cudaMemcpyFromSymbol(status, g_ssd_static_scratch, sizeof(int), lay.off_status);
    if (e != cudaSuccess) return fail(MB200_ERR_LAUNCH, "ssd_static_status: %s", cudaGetErrorString(e));
    return MB200_OK;
}

extern "C" int mb200_ssd_fold_state(const float *s_in, const float *range_decay, const float *s_local, float *s_out,
                                    int64_t rows, int64_t row, int32_t device, void *stream)
{
    using namespace mb200;
    MB200_CHECK_ARG(range_decay && s_local && s_out && rows >= 0 && row > 0, "ssd_fold_state: bad argument");
    if (rows == 0) return MB200_OK;
    if (int rc = enter_device(device)) return rc;
    const int64_t total = rows * row;
    const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
    ssd_fold_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(s_in, range_decay, s_local, s_out, rows, row);
    MB200_CHECK_LAUNCH("ssd_fold_state");
    return MB200_OK;
}

extern "C" int mb200_ssd_fold_ranges(const float *summaries, int64_t record_stride, int32_t first, int32_t last, float *s_out,
                                     int64_t rows, int64_t row, int32_t device, void *stream)
{
    using namespace mb200;
    MB200_CHECK_ARG(summaries && s_out && rows >= 0 && row > 0 && first >= 0 && last >= first && record_stride >= rows * row + rows,
                    "ssd_fold_ranges: bad argument");
    if (rows == 0) return MB200_OK;
    if (int rc = enter_device(device)) return rc;
    const int64_t total = rows * row;
    const int blocks = (int)std::min<int64_t>((total + 255) / 256, 148 * 8);
    ssd_fold_ranges_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(summaries, record_stride, first, last, s_out, rows, row);
    MB200_CHECK_LAUNCH("ssd_fold_ranges");
    return MB200_OK;
}
