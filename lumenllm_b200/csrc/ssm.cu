// Kernels of a selective state-space mixer (a linear recurrence over time with a matrix state
// per head) and of the element-wise pieces around it:
//   - the short causal convolution, with bias and SiLU, of some columns of the input
//     projection, whose last inputs are part of a sequence's state,
//   - the recurrence S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t,
//   - the gate y * silu(z) followed by an RMS norm in equal parts of the row,
//   - xIELU, an activation with two learned numbers.
// All arithmetic is float32 with the precise exponentials. The input projection arrives as the
// S partial sums of a split matrix product, [S, rows, width], which are added in rising order
// of S wherever a value is read. A step brings cu_q[b+1] - cu_q[b] tokens of sequence b (any
// number, also none); state lives in row seq_slot[b] of its store.
#include "common.cuh"

#define SSM_MAX_TAPS 16

__device__ __forceinline__ float sum_parts(const float* p, int S, size_t stride) {
    float x = p[0];
    for (int s = 1; s < S; ++s) x += p[(size_t)s * stride];
    return x;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

// ---------------------------------------------------------------- convolution + bias + SiLU
// out[t, c] = silu(bias[c] + sum_j w[j, c] * in[t - taps + 1 + j, c]) for the C columns of the
// projection that start at column c0; in[] before the step's first token of the sequence comes
// from state[slot][taps - 1 + (t' - first)] (rows oldest to newest, zeros for a new sequence).
// The state is not written here (conv_state_kernel does, after every reader is done).
#define CONV_RUN 8
// TAPS > 0: the number of taps is known when the kernel is compiled (the window then stays in
// registers and the row loop is unrolled); TAPS == 0: any number up to SSM_MAX_TAPS.
template <int TAPS>
__global__ void __launch_bounds__(256)
conv_silu_kernel(const float* __restrict__ u, int S, size_t split_stride, int Wu, int c0, int C,
                 const float* __restrict__ w, const float* __restrict__ bias, int taps_any,
                 const float* __restrict__ state, size_t slot_stride, const int* __restrict__ tok_seq,
                 const int* __restrict__ cu_q, const int* __restrict__ seq_slot, float* __restrict__ out, int N) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t0 = blockIdx.y * CONV_RUN;
    if (c >= C || t0 >= N) return;
    const int taps = TAPS > 0 ? TAPS : taps_any;
    // a thread walks CONV_RUN rows of its channel; the taps - 1 inputs before a row stay in
    // registers from row to row and are fetched anew at the run's first row and wherever a
    // sequence begins
    float win[SSM_MAX_TAPS], wk[SSM_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < SSM_MAX_TAPS; ++j) wk[j] = j < taps ? w[(size_t)j * C + c] : 0.0f;
    const float bc = bias ? bias[c] : 0.0f;
    int b_prev = -1;
    const int t_end = min(t0 + CONV_RUN, N);
#pragma unroll
    for (int t = t0; t < t0 + CONV_RUN; ++t) {
        if (t >= t_end) break;
        const int b = tok_seq[t];
        if (t == t0 || b != b_prev) {
            const int first = cu_q[b];
            const float* st = state + (size_t)seq_slot[b] * slot_stride;
#pragma unroll
            for (int j = 0; j < SSM_MAX_TAPS - 1; ++j)
                if (j < taps - 1) {
                    const int src = t - (taps - 1) + j;
                    win[j] = src >= first ? sum_parts(u + (size_t)src * Wu + c0 + c, S, split_stride)
                                          : st[(size_t)(taps - 1 + src - first) * C + c];
                }
            b_prev = b;
        }
        const float x = sum_parts(u + (size_t)t * Wu + c0 + c, S, split_stride);
        float acc = bc;
#pragma unroll
        for (int j = 0; j < SSM_MAX_TAPS - 1; ++j)
            if (j < taps - 1) acc = fmaf(wk[j], win[j], acc);
#pragma unroll
        for (int j = 0; j < SSM_MAX_TAPS; ++j)
            if (j == taps - 1) acc = fmaf(wk[j], x, acc);
#pragma unroll
        for (int j = 0; j < SSM_MAX_TAPS - 1; ++j)
            if (j < taps - 1) win[j] = (j + 1 < taps - 1) ? win[j + 1] : x;
        out[(size_t)t * C + c] = silu_f(acc);
    }
}

// The state moved on to the end of the step: its rows become the last taps - 1 inputs of the
// sequence, taken from the step's rows and, where the step brought fewer, from the old state.
__global__ void __launch_bounds__(256)
conv_state_kernel(const float* __restrict__ u, int S, size_t split_stride, int Wu, int c0, int C, int taps,
                  float* __restrict__ state, size_t slot_stride, const int* __restrict__ cu_q,
                  const int* __restrict__ seq_slot) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= C) return;
    const int first = cu_q[b], qlen = cu_q[b + 1] - first;
    if (qlen <= 0) return;
    float* st = state + (size_t)seq_slot[b] * slot_stride;
    float v[SSM_MAX_TAPS];
#pragma unroll
    for (int r = 0; r < SSM_MAX_TAPS - 1; ++r) {
        if (r < taps - 1) {
            const int li = qlen - (taps - 1) + r;
            v[r] = li >= 0 ? sum_parts(u + (size_t)(first + li) * Wu + c0 + c, S, split_stride)
                           : st[(size_t)(r + qlen) * C + c];
        }
    }
#pragma unroll
    for (int r = 0; r < SSM_MAX_TAPS - 1; ++r)
        if (r < taps - 1) st[(size_t)r * C + c] = v[r];
}

// One token a sequence (row b is sequence b's): convolution and state in one pass, a thread a
// (sequence, column), which reads the state, uses it and shifts it.
__global__ void __launch_bounds__(256)
conv_silu_decode_kernel(const float* __restrict__ u, int S, size_t split_stride, int Wu, int c0, int C,
                        const float* __restrict__ w, const float* __restrict__ bias, int taps,
                        float* __restrict__ state, size_t slot_stride, const int* __restrict__ seq_slot,
                        float* __restrict__ out, int N) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (c >= C || t >= N) return;
    float* st = state + (size_t)seq_slot[t] * slot_stride;
    const float x = sum_parts(u + (size_t)t * Wu + c0 + c, S, split_stride);
    float acc = bias ? bias[c] : 0.0f;
    float v[SSM_MAX_TAPS];
#pragma unroll
    for (int r = 0; r < SSM_MAX_TAPS - 1; ++r)
        if (r < taps - 1) {
            v[r] = st[(size_t)r * C + c];
            acc = fmaf(w[(size_t)r * C + c], v[r], acc);
        }
    acc = fmaf(w[(size_t)(taps - 1) * C + c], x, acc);
#pragma unroll
    for (int r = 0; r < SSM_MAX_TAPS - 1; ++r)
        if (r < taps - 1) st[(size_t)r * C + c] = (r + 1 < taps - 1) ? v[r + 1] : x;
    out[(size_t)t * C + c] = silu_f(acc);
}

LUMEN_API int lumen_conv_silu(const float* u, int n_split, long long split_stride, int Wu, int c0, int C,
                              const float* w, const float* bias, int taps, float* state, long long slot_stride,
                              const int* tok_seq, const int* cu_q, const int* seq_slot, int n_seqs, int decode,
                              float* out, int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > SSM_MAX_TAPS || n_split < 1 || c0 < 0 || c0 + C > Wu || (taps > 1 && !state))
        return LUMEN_ERR_BAD_ARGUMENT;
    if (N > 65535 || n_seqs > 65535) return LUMEN_ERR_UNSUPPORTED;
    dim3 grid((C + 255) / 256, N);
    if (decode) {
        lumen_launch(conv_silu_decode_kernel, grid, dim3(256), 0, stream, u, n_split, (size_t)split_stride, Wu, c0, C, w,
                     bias, taps, state, (size_t)slot_stride, seq_slot, out, N);
        LUMEN_LAUNCH_CHECK();
        return 0;
    }
    const dim3 cgrid((C + 255) / 256, (N + CONV_RUN - 1) / CONV_RUN);
#define CONV_GO(T_)                                                                                                 \
    lumen_launch(conv_silu_kernel<T_>, cgrid, dim3(256), 0, stream, u, n_split, (size_t)split_stride, Wu, c0, C, w, \
                 bias, taps, (const float*)state, (size_t)slot_stride, tok_seq, cu_q, seq_slot, out, N)
    switch (taps) {
        case 2: CONV_GO(2); break;
        case 3: CONV_GO(3); break;
        case 4: CONV_GO(4); break;
        default: CONV_GO(0); break;
    }
#undef CONV_GO
    LUMEN_LAUNCH_CHECK();
    if (taps > 1) {
        lumen_launch(conv_state_kernel, dim3((C + 255) / 256, n_seqs), dim3(256), 0, stream, u, n_split,
                     (size_t)split_stride, Wu, c0, C, taps, state, (size_t)slot_stride, cu_q, seq_slot);
        LUMEN_LAUNCH_CHECK();
    }
    return 0;
}

// ---------------------------------------------------------------- the recurrence
// A block takes one (sequence, head) and PB of the head's P channels, and walks the sequence's
// tokens of this step in order. Thread (p, j), j < NS, keeps 32 state values S[n, p] in
// registers, n = 4 (j + NS q) + c for q < 8, c < 4 (NS a power of two up to 32, so up to 1,024
// states; places beyond the state's size hold zeros and stay zero): for every token it decays
// them, adds dt B[n] x[p], and sums S[n, p] C[n] over its n in four running sums; the NS
// threads of a channel add their sums by shuffles in a fixed order. Tokens are staged a chunk
// at a time in shared memory (x, B, C of the head's group by asynchronous copies, the next
// chunk's under way while this one is worked on, B and C rows padded with zeros to 32 NS values
// and read four values at a time; and dt and the decay, which the first threads make from the
// projection's dt column: dt = softplus(sum + dt_bias), a = exp(-exp(A_log) dt)). The order of
// every sum depends on the sizes alone, so a token's result is the same however the sequence
// was cut into steps and whatever else is in the batch.
#define SSM_R 32

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int NS>
__global__ void __launch_bounds__(256, 1)
ssm_scan_kernel(const float* __restrict__ xbc, int C, int inner, int H, int P, int Nst, int G,
                const float* __restrict__ u, int S, size_t split_stride, int Wu, int cdt,
                const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dskip,
                float* __restrict__ state, size_t slot_stride, const int* __restrict__ cu_q,
                const int* __restrict__ seq_slot, float* __restrict__ y, int PB, int vec, int chunk) {
    extern __shared__ __align__(16) float sm[];
    constexpr int NP = SSM_R * NS;                   // a staged B or C row, zeros from Nst on
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x, h = blockIdx.y, p0 = blockIdx.z * PB;
    const int first = cu_q[b], qlen = cu_q[b + 1] - first;
    if (qlen <= 0) return;
    const int tid = threadIdx.x, j = tid % NS, pl = tid / NS, p = p0 + pl;
    const bool live = pl < PB && p < P;
    const int g = h / (H / G);
    // two buffers of `chunk` tokens each: [x: chunk x PB | B: chunk x NP | C: chunk x NP | dt | decay]
    const int buf_floats = chunk * (PB + 2 * NP) + 2 * chunk;
    for (int which = 0; which < 2; ++which) {        // the rows' padding, written once
        float* Bs = sm + which * buf_floats + chunk * PB;
        for (int i = tid; i < 2 * chunk * NP; i += blockDim.x)
            if (i % NP >= Nst) Bs[i] = 0.0f;
    }
    float* st = state + (size_t)seq_slot[b] * slot_stride + (size_t)h * Nst * P;
    float s[SSM_R];
#pragma unroll
    for (int r = 0; r < SSM_R; ++r) {
        const int n = 4 * (j + NS * (r >> 2)) + (r & 3);
        s[r] = (live && n < Nst) ? st[(size_t)n * P + p] : 0.0f;
    }
    const float a_h = -expf(A_log[h]), bias_h = dt_bias[h], d_h = Dskip[h];
    // asks for a chunk's x, B and C rows (asynchronous copies into buffer `which`) and returns
    // the raw dt of the token this thread will finish (tid < tokens of the chunk)
    auto request = [&](int t0, int which) -> float {
        float* xs = sm + which * buf_floats;
        float* Bs = xs + chunk * PB;
        float* Cs = Bs + chunk * NP;
        const int nt = min(chunk, qlen - t0);
        if (vec) {
            const int pv = PB >> 2, nv = Nst >> 2;
            for (int i = tid; i < nt * pv; i += blockDim.x) {
                const int tt = i / pv, pp = (i - tt * pv) << 2;
                if (p0 + pp < P) cp_async16(xs + tt * PB + pp, xbc + (size_t)(first + t0 + tt) * C + h * P + p0 + pp);
            }
            for (int i = tid; i < nt * nv; i += blockDim.x) {
                const int tt = i / nv, n = (i - tt * nv) << 2;
                const float* row = xbc + (size_t)(first + t0 + tt) * C + inner + g * Nst + n;
                cp_async16(Bs + tt * NP + n, row);
                cp_async16(Cs + tt * NP + n, row + (size_t)G * Nst);
            }
        } else {
            for (int i = tid; i < nt * PB; i += blockDim.x) {
                const int tt = i / PB, pp = i - tt * PB;
                if (p0 + pp < P) cp_async4(xs + i, xbc + (size_t)(first + t0 + tt) * C + h * P + p0 + pp);
            }
            for (int i = tid; i < nt * Nst; i += blockDim.x) {
                const int tt = i / Nst, n = i - tt * Nst;
                const float* row = xbc + (size_t)(first + t0 + tt) * C + inner + g * Nst + n;
                cp_async4(Bs + tt * NP + n, row);
                cp_async4(Cs + tt * NP + n, row + (size_t)G * Nst);
            }
        }
        cp_async_commit();
        return tid < nt ? sum_parts(u + (size_t)(first + t0 + tid) * Wu + cdt + h, S, split_stride) : 0.0f;
    };
    auto finish = [&](int t0, int which, float raw) {
        float* dts = sm + which * buf_floats + chunk * (PB + 2 * NP);
        if (tid < min(chunk, qlen - t0)) {
            const float dt = softplus_f(raw + bias_h);
            dts[tid] = dt;
            dts[chunk + tid] = expf(a_h * dt);
        }
    };
    float raw = request(0, 0);
    int which = 0;
    for (int t0 = 0; t0 < qlen; t0 += chunk, which ^= 1) {
        const int nt = min(chunk, qlen - t0);
        finish(t0, which, raw);
        cp_async_wait_all();
        __syncthreads();                  // this chunk is in place; everyone is done with the other buffer
        if (t0 + chunk < qlen) raw = request(t0 + chunk, which ^ 1);
        const float* xs = sm + which * buf_floats;
        const float* Bs = xs + chunk * PB;
        const float* Cs = Bs + chunk * NP;
        const float* dts = Cs + chunk * NP;
        const float* decs = dts + chunk;
        for (int tt = 0; tt < nt; ++tt) {
            const float dec = decs[tt], x = live ? xs[tt * PB + pl] : 0.0f, dx = dts[tt] * x;
            const float4* B4 = reinterpret_cast<const float4*>(Bs + tt * NP) + j;
            const float4* C4 = reinterpret_cast<const float4*>(Cs + tt * NP) + j;
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int q = 0; q < SSM_R / 4; ++q) {
                const float4 bv = B4[NS * q], cv = C4[NS * q];
                s[4 * q + 0] = fmaf(dec, s[4 * q + 0], dx * bv.x);
                s[4 * q + 1] = fmaf(dec, s[4 * q + 1], dx * bv.y);
                s[4 * q + 2] = fmaf(dec, s[4 * q + 2], dx * bv.z);
                s[4 * q + 3] = fmaf(dec, s[4 * q + 3], dx * bv.w);
                a0 = fmaf(s[4 * q + 0], cv.x, a0);
                a1 = fmaf(s[4 * q + 1], cv.y, a1);
                a2 = fmaf(s[4 * q + 2], cv.z, a2);
                a3 = fmaf(s[4 * q + 3], cv.w, a3);
            }
            float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
            for (int o = NS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && j == 0) y[(size_t)(first + t0 + tt) * inner + h * P + p] = fmaf(d_h, x, acc);
        }
    }
#pragma unroll
    for (int r = 0; r < SSM_R; ++r) {
        const int n = 4 * (j + NS * (r >> 2)) + (r & 3);
        if (live && n < Nst) st[(size_t)n * P + p] = s[r];
    }
}

// xbc float32 [N, C] with C = inner + 2 G Nst (x, then B, then C of every group); u the input
// projection's partial sums [S, N, Wu], whose columns cdt .. cdt + H - 1 are dt; state float32
// [slots, H, Nst, P]; y float32 [N, inner].
LUMEN_API int lumen_ssm_scan(const float* xbc, int H, int P, int Nst, int G, const float* u, int n_split,
                             long long split_stride, int Wu, int cdt, const float* dt_bias, const float* A_log,
                             const float* Dskip, float* state, long long slot_stride, const int* cu_q,
                             const int* seq_slot, int n_seqs, float* y, int N, cudaStream_t stream) {
    if (N <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || P <= 0 || Nst <= 0 || G <= 0 || H % G || n_split < 1 || cdt < 0 || cdt + H > Wu)
        return LUMEN_ERR_BAD_ARGUMENT;
    if (Nst > 32 * SSM_R || H > 65535) return LUMEN_ERR_UNSUPPORTED;
    int NS = 1;
    while (NS * SSM_R < Nst) NS <<= 1;
    int PB = P < 256 / NS ? P : 256 / NS;      // at most 256 threads a block: the state stays in registers
    // more blocks than SMs where a step has few (sequence, head) pairs: a head's channels are
    // independent of one another, so how they are dealt out changes no result
    while ((long long)n_seqs * H * ((P + PB - 1) / PB) < 2 * 148 && PB * NS > 128 && PB % 2 == 0) PB /= 2;
    const int zb = (P + PB - 1) / PB;
    if (zb > 65535) return LUMEN_ERR_UNSUPPORTED;
    int threads = ((PB * NS + 31) / 32) * 32;
    const int inner = H * P, C = inner + 2 * G * Nst;
    const int chunk = NS * SSM_R <= 512 ? 16 : 8;             // tokens staged at a time
    const size_t smem = 2 * (size_t)(chunk * (PB + 2 * NS * SSM_R) + 2 * chunk) * sizeof(float);
    if (smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    // 16-byte copies where every row piece starts on a 16-byte boundary, else 4-byte ones
    const int vec = (P % 4 == 0 && PB % 4 == 0 && Nst % 4 == 0 && ((uintptr_t)xbc & 15) == 0) ? 1 : 0;
#define SSM_GO(NS_)                                                                                                   \
    case NS_: {                                                                                                       \
        auto k = ssm_scan_kernel<NS_>;                                                                                \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
        lumen_launch(k, dim3(n_seqs, H, zb), dim3(threads), smem, stream, xbc, C, inner, H, P, Nst, G, u, n_split,    \
                     (size_t)split_stride, Wu, cdt, dt_bias, A_log, Dskip, state, (size_t)slot_stride, cu_q,          \
                     seq_slot, y, PB, vec, chunk);                                                                    \
        break;                                                                                                        \
    }
    switch (NS) {
        SSM_GO(1) SSM_GO(2) SSM_GO(4) SSM_GO(8) SSM_GO(16) SSM_GO(32)
        default: return LUMEN_ERR_UNSUPPORTED;
    }
#undef SSM_GO
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- gate, then RMS norm in parts
// v = y * silu(z), z = columns c0 .. c0 + W - 1 of the projection's partial sums; the row is cut
// into `parts` equal pieces, each divided by its own root mean square (eps inside the root) and
// multiplied by w. All threads make the gated values, a warp sums a piece at a time (lanes
// strided over it, then a butterfly: an order that depends on the piece's length alone).
template <typename TOut>
__global__ void __launch_bounds__(1024)
gated_part_norm_kernel(const float* __restrict__ y, const float* __restrict__ u, int S, size_t split_stride, int Wu,
                       int c0, const float* __restrict__ w, float eps, int W, int parts, TOut* __restrict__ out) {
    extern __shared__ __align__(16) float vs[];      // W floats, then one scale a part
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int len = W / parts;
    float* scale = vs + W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float z = sum_parts(u + (size_t)t * Wu + c0 + i, S, split_stride);
        vs[i] = y[(size_t)t * W + i] * silu_f(z);
    }
    __syncthreads();
    for (int g = warp; g < parts; g += nwarp) {
        float ss = 0.0f;
        for (int e = lane; e < len; e += 32) { const float v = vs[g * len + e]; ss += v * v; }
        ss = warp_sum(ss);
        if (lane == 0) scale[g] = 1.0f / sqrtf(ss / (float)len + eps);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)t * W + i] = from_f32<TOut>(vs[i] * scale[i / len] * w[i]);
}

LUMEN_API int lumen_gated_part_norm(const float* y, const float* u, int n_split, long long split_stride, int Wu,
                                    int c0, const float* w, float eps, int W, int parts, void* out, int out_is_bf16,
                                    int N, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (W <= 0 || parts <= 0 || W % parts || n_split < 1 || c0 < 0 || c0 + W > Wu) return LUMEN_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)(W + parts) * sizeof(float);
    if (smem > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    int threads = N >= 2 * 148 ? 256 : ((W + 31) / 32) * 32;     // few rows: wide blocks, all loads in flight
    if (threads > 1024) threads = 1024;
    if (threads < 64) threads = 64;
    if (out_is_bf16) {
        auto k = gated_part_norm_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(N), dim3(threads), smem, stream, y, u, n_split, (size_t)split_stride, Wu, c0, w, eps, W,
                     parts, (__nv_bfloat16*)out);
    } else {
        auto k = gated_part_norm_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        lumen_launch(k, dim3(N), dim3(threads), smem, stream, y, u, n_split, (size_t)split_stride, Wu, c0, w, eps, W,
                     parts, (float*)out);
    }
    LUMEN_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------- xIELU
// z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2, with
// (p, q) = act[0], act[1]. z arrives as partial sums [S, total].
template <typename TOut>
__global__ void xielu_kernel(const float* __restrict__ z, int S, size_t split_stride, const float* __restrict__ act,
                             TOut* __restrict__ out, long long total) {
    pdl_trigger();
    pdl_wait();
    const float ap = softplus_f(act[0]), aq = 0.5f + softplus_f(act[1]);
    const long long step = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const float x = sum_parts(z + i, S, split_stride);
        const float r = x > 0.0f ? fmaf(ap * x, x, 0.5f * x) : fmaf(aq, expm1f(x) - x, 0.5f * x);
        out[i] = from_f32<TOut>(r);
    }
}

LUMEN_API int lumen_xielu(const float* z, int n_split, long long split_stride, const float* act, void* out,
                          int out_is_bf16, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (n_split < 1 || !act) return LUMEN_ERR_BAD_ARGUMENT;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_is_bf16)
        lumen_launch(xielu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, z, n_split, (size_t)split_stride,
                     act, (__nv_bfloat16*)out, total);
    else
        lumen_launch(xielu_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, z, n_split, (size_t)split_stride, act,
                     (float*)out, total);
    LUMEN_LAUNCH_CHECK();
    return 0;
}
