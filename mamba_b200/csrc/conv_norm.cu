// The two element-wise steps either side of the scan in the Mamba mixers, for sm_100a:
//   causal depthwise conv1d (+ SiLU) before the scan -- prefill form and single-token decode form;
//   gated RMSNorm (optionally per group) after the SSD scan.
// Both are pure streaming work (every input read once, every output written once), so the kernels are built
// around 16-byte accesses and keep everything else in registers.
#include <type_traits>

#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kMaxWidth = 4;

__device__ __forceinline__ float act_silu(float v, int activation) { return activation ? v / (1.f + __expf(-v)) : v; }

// A packet of PB bytes (16 or 8) of T, widened to floats and back.
template <typename T, int PB> struct Pkt {
    static constexpr int N = PB / sizeof(T);
    uint32_t w[PB / 4];
    __device__ __forceinline__ void zero()
    {
#pragma unroll
        for (int i = 0; i < PB / 4; ++i) w[i] = 0u;
    }
    __device__ __forceinline__ void load(const T *p)
    {
        if constexpr (PB == 16) {
            const uint4 v = *reinterpret_cast<const uint4 *>(p);
            w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        } else {
            const uint2 v = *reinterpret_cast<const uint2 *>(p);
            w[0] = v.x; w[1] = v.y;
        }
    }
    __device__ __forceinline__ void store(T *p) const
    {
        if constexpr (PB == 16) *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
        else *reinterpret_cast<uint2 *>(p) = make_uint2(w[0], w[1]);
    }
    __device__ __forceinline__ void unpack(float (&f)[N]) const
    {
        const T *e = reinterpret_cast<const T *>(w);
#pragma unroll
        for (int i = 0; i < N; ++i) f[i] = to_float(e[i]);
    }
    __device__ __forceinline__ void pack(const float (&f)[N])
    {
        T *e = reinterpret_cast<T *>(w);
#pragma unroll
        for (int i = 0; i < N; ++i) e[i] = from_float<T>(f[i]);
    }
};

// VEC consecutive parameters (weight or bias) starting at a column that is a multiple of VEC, as floats: one or two
// 16-byte loads when the parameter tensor allows, element loads otherwise.
template <int VEC>
__device__ __forceinline__ void load_params(const void *p, int dtype, bool vec_ok, int col, float (&f)[VEC])
{
    if (vec_ok && dtype == MB200_F32 && VEC % 4 == 0) {
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
            const float4 v = reinterpret_cast<const float4 *>(static_cast<const float *>(p) + col)[q];
            f[4 * q] = v.x; f[4 * q + 1] = v.y; f[4 * q + 2] = v.z; f[4 * q + 3] = v.w;
        }
    } else if (vec_ok && VEC == 8 && dtype == MB200_BF16) {
        Vec16<__nv_bfloat16> v;
        v.load(static_cast<const __nv_bfloat16 *>(p) + col);
        float t[8];
        v.unpack(t);
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = t[i % 8];
    } else if (vec_ok && VEC == 8 && dtype == MB200_F16) {
        Vec16<__half> v;
        v.load(static_cast<const __half *>(p) + col);
        float t[8];
        v.unpack(t);
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = t[i % 8];
    } else if (vec_ok && VEC == 4 && dtype != MB200_F32) {
        const uint2 v = *reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(p) + col);
        const uint32_t ww[2] = {v.x, v.y};
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const uint16_t h = (uint16_t)(ww[(i % 4) >> 1] >> (16 * (i & 1)));
            f[i] = dtype == MB200_BF16 ? __uint_as_float((uint32_t)h << 16) : __half2float(__ushort_as_half(h));
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) f[i] = load_any(p, dtype, col + i);
    }
}

// silu for the element-wise kernels: exact form for fp32 tensors, the single-MUFU tanh form (relative error 2^-11,
// below the rounding step of a 16-bit result) for 16-bit ones
template <typename T> __device__ __forceinline__ float silu_io(float z)
{
    if constexpr (sizeof(T) == 2) return silu_for_bf16(z);
    else return z / (1.f + __expf(-z));
}

// ---- conv1d, channels contiguous (the layout Mamba-2 hands over: a (batch, seqlen, dim) tensor viewed as
// (batch, dim, seqlen)).  A thread owns VEC adjacent channels and walks a segment of the sequence with the last
// width-1 rows of its channels in registers, so every row is read once (plus width-1 rows of halo per segment).
constexpr int kConvSteps = 16;      // output steps per thread of the channels-contiguous kernel
// W (width), packed sequences and the activation are compile-time so that the inner loop holds nothing but loads,
// conversions, packed FMAs and stores; `interior` tiles (no sequence edge, no carried state) skip every bounds test.
template <typename T, int W, bool SID, bool ACT>
__global__ void __launch_bounds__(128, 3) conv1d_cl_kernel(const mb200_conv1d_args a)
{
    constexpr int PB = 16, VEC = PB / sizeof(T), NP = VEC / 2;
    constexpr int TT = kConvSteps, H = W - 1;       // H rows of history before the first output step
    const int c0 = (blockIdx.x * 128 + threadIdx.x) * VEC;
    if (c0 >= a.dim) return;
    const int b = blockIdx.z;
    const int t0 = blockIdx.y * TT;
    const T *x = static_cast<const T *>(a.x) + (int64_t)b * a.x_stride[0] + c0;
    T *out = static_cast<T *>(a.out) + (int64_t)b * a.out_stride[0] + c0;
    const int64_t xs = a.x_stride[2], os = a.out_stride[2];
    const bool interior = t0 >= H && t0 + TT <= a.seqlen;
    // rows t0 - H .. t0 + TT - 1 of my channels: every load is issued before any row is used
    Pkt<T, PB> raw[TT + H];
    if (interior) {
        const T *p = x + (int64_t)(t0 - H) * xs;
#pragma unroll
        for (int r = 0; r < TT + H; ++r, p += xs) raw[r].load(p);
    } else {
#pragma unroll
        for (int r = 0; r < TT + H; ++r) {
            const int t = t0 - H + r;
            raw[r].zero();
            if (t >= 0 && t < a.seqlen) raw[r].load(x + (int64_t)t * xs);
        }
    }
    // the W taps of my VEC channels are VEC * W consecutive parameters
    uint64_t w2[W][NP], bias2[NP];
    {
        const bool wvec = (reinterpret_cast<uintptr_t>(a.bias) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.weight) & 15) == 0 && (VEC * W) % VEC == 0;
        float flat[W][VEC], bias[VEC];
#pragma unroll
        for (int q = 0; q < W; ++q) load_params<VEC>(a.weight, a.w_dtype, wvec, c0 * W + q * VEC, flat[q]);
        if (a.bias) load_params<VEC>(a.bias, a.w_dtype, wvec, c0, bias);
#pragma unroll
        for (int q = 0; q < NP; ++q) {
            bias2[q] = a.bias ? pack2(bias[2 * q], bias[2 * q + 1]) : pack2(0.f, 0.f);
#pragma unroll
            for (int k = 0; k < W; ++k) {
                const int i0 = (2 * q) * W + k, i1 = (2 * q + 1) * W + k;       // parameter index of (channel, tap)
                w2[k][q] = pack2(flat[i0 / VEC][i0 % VEC], flat[i1 / VEC][i1 % VEC]);
            }
        }
    }
    auto unpack_row = [&](const Pkt<T, PB> &r, uint64_t (&o)[NP]) {
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
            for (int q = 0; q < NP; ++q) o[q] = pack2(__uint_as_float(r.w[q] << 16), __uint_as_float(r.w[q] & 0xffff0000u));
        } else {
            float f[VEC];
            r.unpack(f);
#pragma unroll
            for (int q = 0; q < NP; ++q) o[q] = pack2(f[2 * q], f[2 * q + 1]);
        }
    };
    uint64_t win[H][NP];                            // the H rows before the step being formed
#pragma unroll
    for (int j = 0; j < H; ++j) {
        const int t = t0 - H + j;
        if (!interior && t < 0 && a.initial_states) {       // before the sequence: the carried state
            const T *st = static_cast<const T *>(a.initial_states) + (int64_t)b * a.init_stride[0];
#pragma unroll
            for (int q = 0; q < NP; ++q)
                win[j][q] = pack2(to_float(st[(int64_t)(c0 + 2 * q) * a.init_stride[1] + (int64_t)(H + t) * a.init_stride[2]]),
                                  to_float(st[(int64_t)(c0 + 2 * q + 1) * a.init_stride[1] + (int64_t)(H + t) * a.init_stride[2]]));
        } else {
            unpack_row(raw[j], win[j]);
        }
    }
    const int32_t *sid = SID ? a.seq_idx + (int64_t)b * a.seqlen : nullptr;
    const uint64_t half2 = pack2(0.5f, 0.5f);
    T *po = out + (int64_t)t0 * os;
#pragma unroll
    for (int u = 0; u < TT; ++u, po += os) {
        const int t = t0 + u;
        uint64_t cur[NP];
        unpack_row(raw[H + u], cur);
        bool keep[H];                               // taps that reach into another packed sequence contribute nothing
#pragma unroll
        for (int j = 0; j < H; ++j) {
            const int tj = t - H + j;
            keep[j] = !SID || tj < 0 || t >= a.seqlen || sid[tj] == sid[t];
        }
        Pkt<T, PB> o;
#pragma unroll
        for (int q = 0; q < NP; ++q) {
            uint64_t s2 = fma2(w2[H][q], cur[q], bias2[q]);
#pragma unroll
            for (int j = 0; j < H; ++j)
                if (!SID || keep[j]) s2 = fma2(w2[j][q], win[j][q], s2);
            float s0, s1;
            if (ACT && sizeof(T) == 2) {            // silu(s) = h + h tanh(h), h = s / 2 (16-bit results)
                const uint64_t h2 = mul2(s2, half2);
                float h0, h1;
                unpack2(h2, h0, h1);
                s2 = fma2(h2, pack2(tanh_approx(h0), tanh_approx(h1)), h2);
            }
            unpack2(s2, s0, s1);
            if (ACT && sizeof(T) == 4) {
                s0 = silu_io<T>(s0);
                s1 = silu_io<T>(s1);
            }
            if constexpr (sizeof(T) == 2) {
                T *e = reinterpret_cast<T *>(&o.w[q]);
                e[0] = from_float<T>(s0);
                e[1] = from_float<T>(s1);
            } else {
                o.w[2 * q] = __float_as_uint(s0);
                o.w[2 * q + 1] = __float_as_uint(s1);
            }
        }
        if (interior || t < a.seqlen) o.store(po);
#pragma unroll
        for (int j = 0; j + 1 < H; ++j)
#pragma unroll
            for (int q = 0; q < NP; ++q) win[j][q] = win[j + 1][q];
        if (H > 0) {
#pragma unroll
            for (int q = 0; q < NP; ++q) win[H - 1][q] = cur[q];
        }
    }
    if (a.final_states && t0 + TT >= a.seqlen && t0 < a.seqlen) {      // the last width-1 inputs (reaching back into the initial state if need be)
        T *fs = static_cast<T *>(a.final_states) + (int64_t)b * a.final_stride[0];
        for (int j = 0; j < H; ++j) {
            const int t = a.seqlen - H + j;
            for (int i = 0; i < VEC; ++i) {
                T v = from_float<T>(0.f);
                if (t >= 0) v = x[(int64_t)t * xs + i];
                else if (a.initial_states)
                    v = static_cast<const T *>(a.initial_states)[(int64_t)b * a.init_stride[0] + (int64_t)(c0 + i) * a.init_stride[1] + (int64_t)(H + t) * a.init_stride[2]];
                fs[(int64_t)(c0 + i) * a.final_stride[1] + (int64_t)j * a.final_stride[2]] = v;
            }
        }
    }
}

// ---- conv1d, any strides (the Mamba-1 layout, time contiguous, among them): one thread per (channel, run of
// kRun steps); neighbouring threads walk neighbouring runs of the same row, so the row is read in whole sectors.
constexpr int kRun = 8;
template <typename T>
__global__ void __launch_bounds__(256) conv1d_any_kernel(const mb200_conv1d_args a)
{
    constexpr int K = kMaxWidth;
    const int runs = (a.seqlen + kRun - 1) / kRun;
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int r = (int)(idx % runs);
    const int c = (int)(idx / runs);
    const int b = blockIdx.y;
    if (c >= a.dim) return;
    const int W = a.width, lead = K - W;
    float w[K];
#pragma unroll
    for (int k = 0; k < K; ++k) w[k] = k >= lead ? load_any(a.weight, a.w_dtype, (int64_t)c * W + (k - lead)) : 0.f;
    const float bias = a.bias ? load_any(a.bias, a.w_dtype, c) : 0.f;
    const T *x = static_cast<const T *>(a.x) + (int64_t)b * a.x_stride[0] + (int64_t)c * a.x_stride[1];
    T *out = static_cast<T *>(a.out) + (int64_t)b * a.out_stride[0] + (int64_t)c * a.out_stride[1];
    const int32_t *sid = a.seq_idx ? a.seq_idx + (int64_t)b * a.seqlen : nullptr;
    auto at = [&](int t) -> float {
        if (t >= a.seqlen || t < -(W - 1)) return 0.f;
        if (t >= 0) return to_float(x[(int64_t)t * a.x_stride[2]]);
        if (a.initial_states)
            return to_float(static_cast<const T *>(a.initial_states)[(int64_t)b * a.init_stride[0] + (int64_t)c * a.init_stride[1] + (int64_t)(W - 1 + t) * a.init_stride[2]]);
        return 0.f;
    };
    const int t0 = r * kRun;
    float v[kRun + K - 1];                          // v[i] = x[t0 - (K-1) + i]
#pragma unroll
    for (int i = 0; i < kRun + K - 1; ++i) v[i] = at(t0 - (K - 1) + i);
#pragma unroll
    for (int i = 0; i < kRun; ++i) {
        const int t = t0 + i;
        if (t < a.seqlen) {
            float s = bias;
#pragma unroll
            for (int k = 0; k < K; ++k) {
                const int tk = t - (K - 1) + k;     // tap k reads step tk
                if (k >= lead && (!sid || tk < 0 || sid[tk] == sid[t])) s = fmaf(w[k], v[i + k], s);
            }
            out[(int64_t)t * a.out_stride[2]] = from_float<T>(act_silu(s, a.activation));
        }
    }
    if (a.final_states && r == runs - 1) {
        T *fs = static_cast<T *>(a.final_states) + (int64_t)b * a.final_stride[0] + (int64_t)c * a.final_stride[1];
        for (int j = 0; j < W - 1; ++j) fs[(int64_t)j * a.final_stride[2]] = from_float<T>(at(a.seqlen - (W - 1) + j));
    }
}

// ---- decode: one new token per sequence.  conv_state (batch, dim, state_len >= width-1) is shifted left by one
// and the token appended; out = act(bias + sum_k w[k] * window[k]) over the last width-1 old entries and the token.
template <typename T>
__global__ void __launch_bounds__(256) conv1d_update_kernel(const mb200_conv1d_update_args a)
{
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= (int64_t)a.batch * a.dim) return;
    const int b = (int)(idx / a.dim), c = (int)(idx % a.dim);
    const int W = a.width, S = a.state_len;
    T *st = static_cast<T *>(a.conv_state) + (int64_t)b * a.state_stride[0] + (int64_t)c * a.state_stride[1];
    const T xt = static_cast<const T *>(a.x)[(int64_t)b * a.x_stride[0] + (int64_t)c * a.x_stride[1]];
    float s = a.bias ? load_any(a.bias, a.w_dtype, c) : 0.f;
    s = fmaf(load_any(a.weight, a.w_dtype, (int64_t)c * W + W - 1), to_float(xt), s);
    for (int j = 0; j < S; ++j) {                   // every old entry is read once and moved one place to the left
        const T old = st[(int64_t)j * a.state_stride[2]];
        const int k = j - (S - (W - 1));            // old entry j is tap k when it is among the last width-1
        if (k >= 0) s = fmaf(load_any(a.weight, a.w_dtype, (int64_t)c * W + k), to_float(old), s);
        if (j > 0) st[(int64_t)(j - 1) * a.state_stride[2]] = old;
    }
    st[(int64_t)(S - 1) * a.state_stride[2]] = xt;
    static_cast<T *>(a.out)[(int64_t)b * a.out_stride[0] + (int64_t)c * a.out_stride[1]] = from_float<T>(act_silu(s, a.activation));
}

// ---- gated RMSNorm: one CTA per (row, group).  y = x * rstd * weight (+ bias) with the gate silu(z) applied to x
// before the statistics (norm_before_gate = 0) or to y after them (= 1); all arithmetic in fp32.
template <typename T, int PER, bool GATE_AFTER>      // PER 16-byte packets per thread; gate applied after the norm or before it
__global__ void __launch_bounds__(256, 3) rmsnorm_gated_kernel(const mb200_rmsnorm_args a, const int threads, const int wvec)
{
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float red[8];
    const int64_t rowi = blockIdx.x;
    const int g = blockIdx.y;
    const int G = a.group_size;
    const T *x = static_cast<const T *>(a.x) + rowi * a.x_stride + (int64_t)g * G;
    const T *z = a.z ? static_cast<const T *>(a.z) + rowi * a.z_stride + (int64_t)g * G : nullptr;
    T *out = static_cast<T *>(a.out) + rowi * a.out_stride + (int64_t)g * G;
    // every packet of the row is requested before any is used
    Vec16<T> px[PER], pz[PER];
#pragma unroll
    for (int p = 0; p < PER; ++p) {
        const int e = (p * threads + threadIdx.x) * VEC;
        if (e < G) {
            px[p].load(x + e);
            if (z) pz[p].load(z + e);
        }
    }
    float v[PER][VEC];
    float ss = 0.f;
#pragma unroll
    for (int p = 0; p < PER; ++p) {
        const int e = (p * threads + threadIdx.x) * VEC;
        if (e < G) {
            px[p].unpack(v[p]);
            if (z && !GATE_AFTER) {
                float zz[VEC];
                pz[p].unpack(zz);
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[p][i] *= silu_io<T>(zz[i]);
            }
#pragma unroll
            for (int i = 0; i < VEC; ++i) ss = fmaf(v[p][i], v[p][i], ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (threads + 31) / 32; ++i) tot += red[i];
    const float rstd = rsqrtf(tot / (float)G + a.eps);
#pragma unroll
    for (int p = 0; p < PER; ++p) {
        const int e = (p * threads + threadIdx.x) * VEC;
        if (e < G) {
            float y[VEC], wv[VEC];
            load_params<VEC>(a.weight, a.w_dtype, wvec != 0, g * G + e, wv);
#pragma unroll
            for (int i = 0; i < VEC; ++i) y[i] = v[p][i] * rstd * wv[i];
            if (a.bias) {
                load_params<VEC>(a.bias, a.w_dtype, wvec != 0, g * G + e, wv);
#pragma unroll
                for (int i = 0; i < VEC; ++i) y[i] += wv[i];
            }
            if (z && GATE_AFTER) {
                float zz[VEC];
                pz[p].unpack(zz);
#pragma unroll
                for (int i = 0; i < VEC; ++i) y[i] *= silu_io<T>(zz[i]);
            }
            Vec16<T> po;
            po.pack(y);
            po.store(out + e);
        }
    }
}

// general form: any group size and alignment, one warp per (row, group), two passes over the row
template <typename T>
__global__ void __launch_bounds__(32) rmsnorm_gated_any_kernel(const mb200_rmsnorm_args a)
{
    const int64_t rowi = blockIdx.x;
    const int g = blockIdx.y, G = a.group_size, lane = threadIdx.x;
    const T *x = static_cast<const T *>(a.x) + rowi * a.x_stride + (int64_t)g * G;
    const T *z = a.z ? static_cast<const T *>(a.z) + rowi * a.z_stride + (int64_t)g * G : nullptr;
    T *out = static_cast<T *>(a.out) + rowi * a.out_stride + (int64_t)g * G;
    auto gated = [&](int e, float &gate) {
        float v = to_float(x[e]);
        gate = 1.f;
        if (z) {
            const float zz = to_float(z[e]);
            gate = zz / (1.f + __expf(-zz));
            if (!a.norm_before_gate) v *= gate;
        }
        return v;
    };
    float ss = 0.f, gate;
    for (int e = lane; e < G; e += 32) {
        const float v = gated(e, gate);
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / (float)G + a.eps);
    for (int e = lane; e < G; e += 32) {
        const float v = gated(e, gate);
        float y = v * rstd * load_any(a.weight, a.w_dtype, g * G + e);
        if (a.bias) y += load_any(a.bias, a.w_dtype, g * G + e);
        if (z && a.norm_before_gate) y *= gate;
        out[e] = from_float<T>(y);
    }
}

bool valid_dtype(int d) { return d == MB200_F32 || d == MB200_F16 || d == MB200_BF16; }
bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
int launch_conv1d(const mb200_conv1d_args &a, cudaStream_t stream)
{
    constexpr int VEC = 16 / sizeof(T);
    const bool channels_last = a.x_stride[1] == 1 && a.out_stride[1] == 1 && a.dim % VEC == 0 && aligned16(a.x) && aligned16(a.out) &&
                               a.x_stride[0] % VEC == 0 && a.x_stride[2] % VEC == 0 && a.out_stride[0] % VEC == 0 && a.out_stride[2] % VEC == 0 &&
                               (a.seqlen + kConvSteps - 1) / kConvSteps <= 65535;
    if (channels_last) {
        const dim3 grid((a.dim / VEC + 127) / 128, (a.seqlen + kConvSteps - 1) / kConvSteps, a.batch);
        auto go = [&](auto w_tag) {
            constexpr int W = decltype(w_tag)::value;
            if (a.seq_idx) {
                if (a.activation) conv1d_cl_kernel<T, W, true, true><<<grid, 128, 0, stream>>>(a);
                else conv1d_cl_kernel<T, W, true, false><<<grid, 128, 0, stream>>>(a);
            } else {
                if (a.activation) conv1d_cl_kernel<T, W, false, true><<<grid, 128, 0, stream>>>(a);
                else conv1d_cl_kernel<T, W, false, false><<<grid, 128, 0, stream>>>(a);
            }
        };
        if (a.width == 4) go(std::integral_constant<int, 4>{});
        else if (a.width == 3) go(std::integral_constant<int, 3>{});
        else go(std::integral_constant<int, 2>{});
    } else {
        const int64_t work = (int64_t)a.dim * ((a.seqlen + kRun - 1) / kRun);
        conv1d_any_kernel<T><<<dim3((unsigned)((work + 255) / 256), a.batch), 256, 0, stream>>>(a);
    }
    return MB200_OK;
}

template <typename T>
int launch_rmsnorm(const mb200_rmsnorm_args &a, cudaStream_t stream)
{
    constexpr int VEC = 16 / sizeof(T);
    const int G = a.group_size, ngroups = a.ncols / G;
    const bool vec_ok = G % VEC == 0 && aligned16(a.x) && aligned16(a.out) && (!a.z || aligned16(a.z)) && a.x_stride % VEC == 0 &&
                        a.out_stride % VEC == 0 && (!a.z || a.z_stride % VEC == 0) && G <= 256 * 4 * VEC;
    dim3 grid((unsigned)a.nrows, ngroups);
    if (!vec_ok) {
        rmsnorm_gated_any_kernel<T><<<grid, 32, 0, stream>>>(a);
        return MB200_OK;
    }
    const int packets = G / VEC;
    int threads = 32;
    while (threads < 256 && threads * 2 <= packets) threads *= 2;      // a packet or two per thread while the group allows
    const int per = (packets + threads - 1) / threads;
    const int wvec = aligned16(a.weight) && (!a.bias || aligned16(a.bias)) ? 1 : 0;      // columns are multiples of VEC: parameter packets are aligned too
    auto go = [&](auto per_tag) {
        constexpr int P = decltype(per_tag)::value;
        if (a.norm_before_gate) rmsnorm_gated_kernel<T, P, true><<<grid, threads, 0, stream>>>(a, threads, wvec);
        else rmsnorm_gated_kernel<T, P, false><<<grid, threads, 0, stream>>>(a, threads, wvec);
    };
    if (per <= 1) go(std::integral_constant<int, 1>{});
    else if (per <= 2) go(std::integral_constant<int, 2>{});
    else go(std::integral_constant<int, 4>{});
    return MB200_OK;
}

}  // namespace
}  // namespace mb200

extern "C" int mb200_causal_conv1d_fwd(const mb200_conv1d_args *args, void *stream_)
{
    using namespace mb200;
    if (!args) return fail(MB200_ERR_BAD_ARG, "causal_conv1d_fwd: args is NULL");
    const mb200_conv1d_args &a = *args;
    MB200_CHECK_ARG(a.batch >= 0 && a.dim > 0 && a.seqlen >= 0, "causal_conv1d_fwd: bad sizes (batch %d dim %d seqlen %d)", a.batch, a.dim, a.seqlen);
    MB200_CHECK_ARG(a.width >= 2 && a.width <= kMaxWidth, "causal_conv1d only supports width between 2 and 4");
    MB200_CHECK_ARG(valid_dtype(a.io_dtype) && valid_dtype(a.w_dtype), "causal_conv1d_fwd: unknown dtype code");
    MB200_CHECK_ARG(a.activation == 0 || a.activation == 1, "causal_conv1d_fwd: activation must be 0 (none) or 1 (silu)");
    MB200_CHECK_ARG(a.batch <= 65535, "causal_conv1d_fwd: batch must be <= 65535");
    if (a.batch == 0 || a.seqlen == 0) return MB200_OK;
    MB200_CHECK_ARG(a.x && a.weight && a.out, "causal_conv1d_fwd: a required tensor is NULL");
    if (int rc = enter_device(a.device)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc;
    if (a.io_dtype == MB200_F32) rc = launch_conv1d<float>(a, stream);
    else if (a.io_dtype == MB200_BF16) rc = launch_conv1d<__nv_bfloat16>(a, stream);
    else rc = launch_conv1d<__half>(a, stream);
    if (rc) return rc;
    MB200_CHECK_LAUNCH("causal_conv1d_fwd");
    return MB200_OK;
}

extern "C" int mb200_causal_conv1d_update(const mb200_conv1d_update_args *args, void *stream_)
{
    using namespace mb200;
    if (!args) return fail(MB200_ERR_BAD_ARG, "causal_conv1d_update: args is NULL");
    const mb200_conv1d_update_args &a = *args;
    MB200_CHECK_ARG(a.batch >= 0 && a.dim > 0, "causal_conv1d_update: bad sizes (batch %d dim %d)", a.batch, a.dim);
    MB200_CHECK_ARG(a.width >= 2 && a.width <= kMaxWidth, "causal_conv1d only supports width between 2 and 4");
    MB200_CHECK_ARG(a.state_len >= a.width - 1, "causal_conv1d_update: conv_state must hold at least width - 1 steps");
    MB200_CHECK_ARG(valid_dtype(a.io_dtype) && valid_dtype(a.w_dtype), "causal_conv1d_update: unknown dtype code");
    if (a.batch == 0) return MB200_OK;
    MB200_CHECK_ARG(a.x && a.weight && a.out && a.conv_state, "causal_conv1d_update: a required tensor is NULL");
    if (int rc = enter_device(a.device)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const unsigned blocks = (unsigned)(((int64_t)a.batch * a.dim + 255) / 256);
    if (a.io_dtype == MB200_F32) conv1d_update_kernel<float><<<blocks, 256, 0, stream>>>(a);
    else if (a.io_dtype == MB200_BF16) conv1d_update_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(a);
    else conv1d_update_kernel<__half><<<blocks, 256, 0, stream>>>(a);
    MB200_CHECK_LAUNCH("causal_conv1d_update");
    return MB200_OK;
}

extern "C" int mb200_rmsnorm_gated_fwd(const mb200_rmsnorm_args *args, void *stream_)
{
    using namespace mb200;
    if (!args) return fail(MB200_ERR_BAD_ARG, "rmsnorm_gated_fwd: args is NULL");
    const mb200_rmsnorm_args &a = *args;
    MB200_CHECK_ARG(a.nrows >= 0 && a.ncols > 0 && a.group_size > 0, "rmsnorm_gated_fwd: bad sizes (rows %lld cols %d group %d)", (long long)a.nrows,
                    a.ncols, a.group_size);
    MB200_CHECK_ARG(a.ncols % a.group_size == 0, "rmsnorm_gated_fwd: the row length must be a multiple of group_size");
    MB200_CHECK_ARG(valid_dtype(a.io_dtype) && valid_dtype(a.w_dtype), "rmsnorm_gated_fwd: unknown dtype code");
    MB200_CHECK_ARG(a.nrows <= 2147483647LL && a.ncols / a.group_size <= 65535, "rmsnorm_gated_fwd: too many rows or groups");
    if (a.nrows == 0) return MB200_OK;
    MB200_CHECK_ARG(a.x && a.weight && a.out, "rmsnorm_gated_fwd: a required tensor is NULL");
    if (int rc = enter_device(a.device)) return rc;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc;
    if (a.io_dtype == MB200_F32) rc = launch_rmsnorm<float>(a, stream);
    else if (a.io_dtype == MB200_BF16) rc = launch_rmsnorm<__nv_bfloat16>(a, stream);
    else rc = launch_rmsnorm<__half>(a, stream);
    if (rc) return rc;
    MB200_CHECK_LAUNCH("rmsnorm_gated_fwd");
    return MB200_OK;
}
