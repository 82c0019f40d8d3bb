// Attention whose softmax weights are mixed ACROSS heads before they meet the values
// ("talking heads" after the softmax), over the paged cache, with a sliding window that keeps
// the first tokens of a sequence in sight:
//
//   a query at position p sees key j if j <= p and (p - j < size or j < keep);
//   w_g(j) = softmax_j(scale * q_g . k_kv(g)(j)) over the visible keys, per head g;
//   m_h(j) = sum_g T[h][g] w_g(j);          out_h = sum_j m_h(j) v_kv(h)(j).
//
// The mix needs every head's NORMALISED weights at a (query, key) pair, so the weights cannot
// stay inside one head's running softmax as in flash attention. The work is cut into three
// phases around a float32 scratch matrix W[token][head][column]:
//   1. scores:  W = scale * q . k                       (per head, keys in parallel)
//   2. softmax over a token's columns per head, then the mix over heads at every column
//   3. values:  out_h = sum over columns of m_h * v     (per head, keys in parallel)
// In steps of prompts (bfloat16) the three are three kernels, 1 and 3 on the tensor cores, 2 in
// place (W becomes m). Otherwise 2 is done by the values kernel itself, for its own columns: the
// scores kernel leaves every 64-column chunk's maximum and sum of exponentials, from which any
// block has all heads' normalisers in a few loads.
// Column c of a token stands for key c if c < kept, else key lo + (c - kept), with
// lo = max(0, p - size + 1) and kept = min(keep, lo): the kept first keys, then the window.
// A token has kept + p - lo + 1 columns; the matrix's row stride is the most any token of the
// step can have. Key and value tiles may have different widths (d, dv). All sums are float32
// and their order depends on the query's own position only, never on the batch. T is float
// (32-bit path) or __nv_bfloat16; scores, weights and the mix are float32 in both.
#include "common.cuh"
#include "mma_utils.cuh"

struct Sight {
    int lo, kept, n;
};
__device__ __forceinline__ Sight sight_of(int p, int size, int keep) {
    Sight s;
    s.lo = (size > 0 && p - size + 1 > 0) ? p - size + 1 : 0;
    s.kept = keep < s.lo ? keep : s.lo;
    if (s.kept < 0) s.kept = 0;
    s.n = s.kept + p - s.lo + 1;
    return s;
}
__device__ __forceinline__ int key_of(const Sight& s, int c) { return c < s.kept ? c : s.lo + (c - s.kept); }

__device__ __forceinline__ void load8(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(b[k]);
        v[2 * k] = f.x;
        v[2 * k + 1] = f.y;
    }
}

// ---------------------------------------------------------------- 1. scores
// Block (token n, kv head g, chunk of TS_COLS columns). The queries of the kv head's `per`
// heads lie in shared memory as float32; four lanes share a key (each takes every fourth
// group of eight values of its row), so a warp walks eight keys at a time.
#define TS_THREADS 128
#define TS_COLS 64
#define TS_MAX_PER 16
template <typename T>
__global__ void __launch_bounds__(TS_THREADS)
talk_scores_kernel(const T* __restrict__ q, const T* __restrict__ kcache, const int* __restrict__ table,
                   int table_stride, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                   float* __restrict__ W, float* __restrict__ stats, int row_stride, int n0, int H, int G, int d,
                   int size, int keep, float scale, int layout, int hsplit) {
    extern __shared__ __align__(16) float qs[];   // per * d floats, then per * TS_COLS scores
    pdl_trigger();       // the kernel behind may come to rest and wait; it still waits for this one's end
    pdl_wait();
    // blockIdx.y counts (kv head, part of its heads): a kv head with more than TS_MAX_PER heads is
    // taken by `hsplit` blocks, each with an equal share of the heads
    const int n = n0 + blockIdx.x, g = blockIdx.y / hsplit, c0 = blockIdx.z * TS_COLS;
    const Sight s = sight_of(tok_pos[n], size, keep);
    if (c0 >= s.n) return;
    const int per = H / G / hsplit;
    const int h0 = g * (H / G) + (blockIdx.y % hsplit) * per;       // the block's first head
    float* sc = qs + per * d;
    const T* qrow = q + ((size_t)n * H + h0) * d;
    for (int e = threadIdx.x; e < per * d; e += TS_THREADS) qs[e] = to_f32(qrow[e]);
    for (int e = threadIdx.x; e < per * TS_COLS; e += TS_THREADS) sc[e] = -INFINITY;
    __syncthreads();
    const int* bt = table + (size_t)tok_seq[n] * table_stride;
    const int sub = threadIdx.x & 3;
    const bool vec = (d & 7) == 0 && layout == LUMEN_LAYOUT_LINEAR;
#pragma unroll
    for (int cc = threadIdx.x >> 2; cc < TS_COLS; cc += TS_THREADS / 4) {
        const int c = c0 + cc;
        const bool live = c < s.n;       // every lane stays for the exchanges below
        const int j = key_of(s, live ? c : s.n - 1);
        const T* tile = kcache + ((size_t)bt[j / LUMEN_PAGE] * G + g) * LUMEN_PAGE * d;
        const int r = j % LUMEN_PAGE;
        float acc[TS_MAX_PER];
#pragma unroll
        for (int hh = 0; hh < TS_MAX_PER; ++hh) acc[hh] = 0.0f;
        if (vec) {
            const T* krow = tile + (size_t)r * d;
            for (int e = sub * 8; e < d; e += 32) {
                float kv[8];
                load8(krow + e, kv);
#pragma unroll
                for (int hh = 0; hh < TS_MAX_PER; ++hh)
                    if (hh < per) {
                        const float4 q0 = *reinterpret_cast<const float4*>(qs + hh * d + e);
                        const float4 q1 = *reinterpret_cast<const float4*>(qs + hh * d + e + 4);
                        float a = acc[hh];
                        a = fmaf(q0.x, kv[0], a); a = fmaf(q0.y, kv[1], a); a = fmaf(q0.z, kv[2], a); a = fmaf(q0.w, kv[3], a);
                        a = fmaf(q1.x, kv[4], a); a = fmaf(q1.y, kv[5], a); a = fmaf(q1.z, kv[6], a); a = fmaf(q1.w, kv[7], a);
                        acc[hh] = a;
                    }
            }
        } else {
            for (int e = sub; e < d; e += 4) {
                const float kv = to_f32(tile[tile_offset(layout, r, e, d)]);
#pragma unroll
                for (int hh = 0; hh < TS_MAX_PER; ++hh)
                    if (hh < per) acc[hh] = fmaf(qs[hh * d + e], kv, acc[hh]);
            }
        }
#pragma unroll
        for (int hh = 0; hh < TS_MAX_PER; ++hh)
            if (hh < per) {
                float a = acc[hh];
                a += __shfl_xor_sync(0xffffffffu, a, 1);
                a += __shfl_xor_sync(0xffffffffu, a, 2);
                if (sub == 0 && live) {
                    W[((size_t)(n - n0) * H + h0 + hh) * row_stride + c] = a * scale;
                    sc[hh * TS_COLS + cc] = a * scale;
                }
            }
    }
    // the chunk's maximum and sum of exponentials per head, for the mix kernel to put together
    __syncthreads();
    const int lane = threadIdx.x & 31, chunks = gridDim.z;
    for (int hh = threadIdx.x >> 5; hh < per; hh += TS_THREADS / 32) {
        const float a = sc[hh * TS_COLS + lane], b = sc[hh * TS_COLS + 32 + lane];
        const float m = warp_max(fmaxf(a, b));
        const float l = warp_sum(expf(a - m) + expf(b - m));      // columns beyond the token's give exp(-inf) = 0
        if (lane == 0) {
            float* st = stats + (((size_t)(n - n0) * H + h0 + hh) * chunks + blockIdx.z) * 2;
            st[0] = m;
            st[1] = l;
        }
    }
}

// ---------------------------------------------------------------- 2. softmax and mix (prompt steps)
// Block = token. First every head's maximum and sum over the token's columns (a warp a head),
// then, 256 columns at a time: every head's weight at the column, and from those each output
// head's mix, written as bfloat16 over the front half of the head's float32 row (the tensor-core
// values kernel reads them so): column c then lands on the bytes of the float32 columns c / 2,
// which belong to this or an earlier group of 256 columns, all read before the barrier.
// Exponentials are the fast form, as in the library's other serving attention kernels (this
// kernel runs in bfloat16 prompt steps only; everywhere else the values kernel mixes, with expf).
// HR > 0 (at least the number of heads, a multiple of 4): a thread keeps its column's weights of
// all heads in registers and reads the talk matrix four values at a time; HR = 0: any number of
// heads, the weights go through shared memory.
#define TM_THREADS 256
#define TM_MAX_H 128
template <int HR>
__global__ void __launch_bounds__(TM_THREADS)
talk_softmax_mix_kernel(float* __restrict__ W, int row_stride, const int* __restrict__ tok_pos, int n0,
                        const float* __restrict__ talk, int H, int size, int keep) {
    extern __shared__ __align__(16) float sm[];   // the talk matrix; with HR = 0 also H * TM_THREADS weights
    __shared__ float mx[TM_MAX_H], inv[TM_MAX_H];
    float* tk = sm;
    float* ws = sm + H * H;                   // used with HR = 0 only
    const int tw = HR > 0 ? HR : H;           // width of a row of the talk matrix in shared memory
    for (int i = threadIdx.x; i < H * tw; i += TM_THREADS) {
        const int hh = i / tw, g = i - hh * tw;
        tk[i] = g < H ? talk[hh * H + g] : 0.0f;                              // never changes
    }
    pdl_trigger();       // the kernel behind may come to rest and wait; it still waits for this one's end
    pdl_wait();
    const int n = blockIdx.x;
    const Sight s = sight_of(tok_pos[n0 + n], size, keep);
    float* rows = W + (size_t)n * H * row_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int g = warp; g < H; g += TM_THREADS / 32) {
        const float* row = rows + (size_t)g * row_stride;
        float m = -INFINITY, l = 0.0f;
        for (int c = lane; c < s.n; c += 32) m = fmaxf(m, row[c]);
        m = warp_max(m);
        for (int c = lane; c < s.n; c += 32) l += __expf(row[c] - m);
        l = warp_sum(l);
        if (lane == 0) {
            mx[g] = m;
            inv[g] = 1.0f / l;
        }
    }
    __syncthreads();
    for (int c0 = 0; c0 < s.n; c0 += TM_THREADS) {
        const int c = c0 + threadIdx.x;
        float p[HR > 0 ? HR : 1];
        if (c < s.n) {
            if (HR > 0) {
#pragma unroll
                for (int g = 0; g < HR; ++g)
                    p[g] = g < H ? __expf(rows[(size_t)g * row_stride + c] - mx[g]) * inv[g] : 0.0f;
            } else {
                for (int g = 0; g < H; ++g)
                    ws[g * TM_THREADS + threadIdx.x] = __expf(rows[(size_t)g * row_stride + c] - mx[g]) * inv[g];
            }
        }
        __syncthreads();             // the narrow stores below land on other threads' scores
        if (c < s.n)
            for (int h = 0; h < H; ++h) {
                float a = 0.0f;
                if (HR > 0) {
                    // the talk matrix lies in rows of HR values (zeros behind the heads)
                    const float4* t4 = reinterpret_cast<const float4*>(tk + h * HR);
#pragma unroll
                    for (int g4 = 0; g4 < HR / 4; ++g4) {
                        const float4 w = t4[g4];
                        a = fmaf(w.x, p[4 * g4], a);
                        a = fmaf(w.y, p[4 * g4 + 1], a);
                        a = fmaf(w.z, p[4 * g4 + 2], a);
                        a = fmaf(w.w, p[4 * g4 + 3], a);
                    }
                } else {
                    const float* t = tk + h * H;
                    for (int g = 0; g < H; ++g) a = fmaf(t[g], ws[g * TM_THREADS + threadIdx.x], a);
                }
                reinterpret_cast<__nv_bfloat16*>(rows + (size_t)h * row_stride)[c] = __float2bfloat16_rn(a);
            }
    }
}

static void launch_mix(int n_rows, cudaStream_t stream, float* W, int row_stride, const int* tok_pos, int n0,
                       const float* talk, int H, int size, int keep) {
#define LUMEN_MIX(HR_, SMEM_)                                                                                          \
    do {                                                                                                               \
        auto k = talk_softmax_mix_kernel<HR_>;                                                                         \
        const size_t smem = (SMEM_);                                                                                   \
        if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
        lumen_launch(k, dim3(n_rows), dim3(TM_THREADS), smem, stream, W, row_stride, tok_pos, n0, talk, H, size, keep); \
    } while (0)
    if (H <= 8) LUMEN_MIX(8, (size_t)H * 8 * sizeof(float));
    else if (H <= 16) LUMEN_MIX(16, (size_t)H * 16 * sizeof(float));
    else if (H <= 32) LUMEN_MIX(32, (size_t)H * 32 * sizeof(float));
    else LUMEN_MIX(0, ((size_t)H * H + (size_t)H * TM_THREADS) * sizeof(float));
#undef LUMEN_MIX
}

// ---------------------------------------------------------------- 3. values
// Block (token n, head h, part z of the columns): eight warps take the part's columns in
// turn, a lane holds dv / 32 values of the output (up to eight); the warps' sums are added in
// warp order. With one part the result goes out as T; with several, float32 partial results
// [part][token][head][dv] that talk_parts_kernel adds in rising order.
#define TV_THREADS 256
#define TV_PART 128
#define TV_MAX_PER 16
// A lane's share of a value row: E consecutive values (E = 4 for values of up to 128, else 8).
template <typename T, int E>
__device__ __forceinline__ void load_vals(const T* p, float* v) {
#pragma unroll
    for (int k = 0; k < E; ++k) v[k] = to_f32(p[k]);
}
template <>
__device__ __forceinline__ void load_vals<__nv_bfloat16, 4>(const __nv_bfloat16* p, float* v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <>
__device__ __forceinline__ void load_vals<float, 4>(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
}

template <typename T, int E, int PER>
__global__ void __launch_bounds__(TV_THREADS)
talk_values_kernel(const float* __restrict__ W, const float* __restrict__ stats, int chunks,
                   const float* __restrict__ talk, int row_stride, const T* __restrict__ vcache,
                   const int* __restrict__ table, int table_stride, const int* __restrict__ tok_seq,
                   const int* __restrict__ tok_pos, T* __restrict__ out, float* __restrict__ parts, int n0, int n_rows,
                   int H, int G, int dv, int size, int keep, int layout, int hsplit) {
    // [warps][per][32 * E] sums | [2][per][TV_PART] mixed weights | [per][H] talk rows | [H] maxima | [H] 1 / sums
    extern __shared__ __align__(16) float acc_s[];
    pdl_trigger();       // the kernel behind may come to rest and wait; it still waits for this one's end
    // the talk matrix never changes: the rows of the block's heads are fetched before the wait
    {
        const int per_ = H / G / hsplit;
        const int h0_ = (blockIdx.y / hsplit) * (H / G) + (blockIdx.y % hsplit) * per_;
        float* tkr_ = acc_s + (TV_THREADS / 32) * per_ * 32 * E + 2 * per_ * TV_PART;
        for (int i = threadIdx.x; i < per_ * H; i += TV_THREADS) tkr_[i] = talk[(size_t)h0_ * H + i];
    }
    pdl_wait();
    const int n = blockIdx.x, g = blockIdx.y / hsplit, z = blockIdx.z;
    const int per = H / G / hsplit;
    const int h0 = g * (H / G) + (blockIdx.y % hsplit) * per;       // the block's first head
    const Sight s = sight_of(tok_pos[n0 + n], size, keep);
    const int c_lo = z * TV_PART, c_hi = min(s.n, c_lo + TV_PART);
    if (c_lo >= s.n) return;             // talk_parts_kernel reads only the parts a token has
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int* bt = table + (size_t)tok_seq[n0 + n] * table_stride;
    // the pages and rows of the warp's columns are asked for now and used behind the mix
    constexpr int COLS = TV_PART / (TV_THREADS / 32);
    int my_page = 0, my_r = 0;
    {
        const int c = c_lo + warp + (TV_THREADS / 32) * lane;
        if (lane < COLS && c < c_hi) {
            const int j = key_of(s, c);
            my_page = bt[j / LUMEN_PAGE];
            my_r = j % LUMEN_PAGE;
        }
    }
    // Softmax and mix for the block's own columns (W holds the scores of ALL heads; the scores
    // kernel left every 64-column chunk's maximum and sum of exponentials in `stats`): first each
    // head's maximum and sum over the token's columns, then at each of the block's columns every
    // head's weight and, from those, the mix for the block's heads, into shared memory.
    float* wmix = acc_s + (TV_THREADS / 32) * per * 32 * E;
    const float* tkr = wmix + 2 * per * TV_PART;
    float* mx = wmix + 2 * per * TV_PART + per * H;
    float* inv = mx + H;
    for (int g2 = warp; g2 < H; g2 += TV_THREADS / 32) {
        const float* st = stats + ((size_t)n * H + g2) * chunks * 2;
        const int used = (s.n + TS_COLS - 1) / TS_COLS;
        float m = -INFINITY, l = 0.0f;
        for (int c = lane; c < used; c += 32) m = fmaxf(m, st[2 * c]);
        m = warp_max(m);
        for (int c = lane; c < used; c += 32) l += st[2 * c + 1] * expf(st[2 * c] - m);
        l = warp_sum(l);
        if (lane == 0) {
            mx[g2] = m;
            inv[g2] = 1.0f / l;
        }
    }
    __syncthreads();
    {
        // thread t: column t % TV_PART; the two halves of the block share the heads whose weights
        // enter the mix (each half its own sum, added when the weights are taken below)
        const int cc = threadIdx.x % TV_PART, c = c_lo + cc, half = threadIdx.x / TV_PART;
        constexpr int HALVES = TV_THREADS / TV_PART;
        const int share = (H + HALVES - 1) / HALVES, g_lo = half * share, g_hi = min(H, g_lo + share);
        if (c < c_hi) {
            float a[PER];
#pragma unroll
            for (int hh = 0; hh < PER; ++hh) a[hh] = 0.0f;
            const float* col = W + (size_t)n * H * row_stride + c;
            for (int g2 = g_lo; g2 < g_hi; ++g2) {
                const float pw = expf(col[(size_t)g2 * row_stride] - mx[g2]) * inv[g2];
#pragma unroll
                for (int hh = 0; hh < PER; ++hh)
                    if (hh < per) a[hh] = fmaf(tkr[hh * H + g2], pw, a[hh]);
            }
#pragma unroll
            for (int hh = 0; hh < PER; ++hh)
                if (hh < per) wmix[(half * per + hh) * TV_PART + cc] = a[hh];
        }
    }
    __syncthreads();
    const int e0 = lane * E;
    const bool mine = e0 < dv;
    const bool whole = layout == LUMEN_LAYOUT_LINEAR && dv % E == 0;      // a lane's values move as one piece
    float acc[PER][E];
#pragma unroll
    for (int hh = 0; hh < PER; ++hh)
#pragma unroll
        for (int k = 0; k < E; ++k) acc[hh][k] = 0.0f;
    // Lane l fetches, for the warp's l-th column, the page and row of its key and the heads'
    // weights; the walk below takes them from there, so that no load in it waits for another.
    float my_w[PER];
#pragma unroll
    for (int hh = 0; hh < PER; ++hh) my_w[hh] = 0.0f;
    {
        const int c = c_lo + warp + (TV_THREADS / 32) * lane;
        if (lane < COLS && c < c_hi) {
#pragma unroll
            for (int hh = 0; hh < PER; ++hh)
                if (hh < per) my_w[hh] = wmix[hh * TV_PART + (c - c_lo)] + wmix[(per + hh) * TV_PART + (c - c_lo)];
        }
    }
#pragma unroll 4
    for (int k = 0; k < COLS; ++k) {
        if (c_lo + warp + (TV_THREADS / 32) * k >= c_hi) break;          // the same for the whole warp
        const int page = __shfl_sync(0xffffffffu, my_page, k), r = __shfl_sync(0xffffffffu, my_r, k);
        const T* tile = vcache + ((size_t)page * G + g) * LUMEN_PAGE * dv;
        float v[E];
        if (!mine) {
#pragma unroll
            for (int e = 0; e < E; ++e) v[e] = 0.0f;
        } else if (whole) {
            load_vals<T, E>(tile + (size_t)r * dv + e0, v);
        } else {
#pragma unroll
            for (int e = 0; e < E; ++e) v[e] = e0 + e < dv ? to_f32(tile[tile_offset(layout, r, e0 + e, dv)]) : 0.0f;
        }
#pragma unroll
        for (int hh = 0; hh < PER; ++hh) {
            const float w = __shfl_sync(0xffffffffu, my_w[hh], k);
            if (hh < per) {
#pragma unroll
                for (int e = 0; e < E; ++e) acc[hh][e] = fmaf(w, v[e], acc[hh][e]);
            }
        }
    }
    const int width = 32 * E;
#pragma unroll
    for (int hh = 0; hh < PER; ++hh)
        if (hh < per)
#pragma unroll
            for (int k = 0; k < E; ++k) acc_s[((size_t)warp * per + hh) * width + e0 + k] = acc[hh][k];
    __syncthreads();
    for (int i = threadIdx.x; i < per * dv; i += TV_THREADS) {
        const int hh = i / dv, e = i - hh * dv;
        float a = 0.0f;
#pragma unroll
        for (int w8 = 0; w8 < TV_THREADS / 32; ++w8) a += acc_s[((size_t)w8 * per + hh) * width + e];
        const int h = h0 + hh;
        if (parts) parts[(((size_t)z * n_rows + n) * H + h) * dv + e] = a;
        else out[((size_t)(n0 + n) * H + h) * dv + e] = from_f32<T>(a);
    }
}

template <typename T, int E>
static void launch_values(int per, dim3 grid, size_t smem, cudaStream_t stream, const float* W, const float* stats,
                          int chunks, const float* talk, int row_stride, const T* vc, const int* table, int table_stride, const int* tok_seq, const int* tok_pos,
                          T* out, float* parts, int n0, int rows, int H, int G, int dv, int size, int keep, int layout,
                          int hsplit) {
#define LUMEN_TV(PER_)                                                                                               \
    lumen_launch(talk_values_kernel<T, E, PER_>, grid, dim3(TV_THREADS), smem, stream, W, stats, chunks, talk,       \
                 row_stride, vc, table,                                                                              \
                 table_stride, tok_seq, tok_pos, out, parts, n0, rows, H, G, dv, size, keep, layout, hsplit)
    if (per <= 1) LUMEN_TV(1);
    else if (per <= 2) LUMEN_TV(2);
    else if (per <= 4) LUMEN_TV(4);
    else if (per <= 8) LUMEN_TV(8);
    else LUMEN_TV(16);
#undef LUMEN_TV
}

template <typename T>
__global__ void talk_parts_kernel(const float* __restrict__ parts, int Z, size_t part_stride,
                                  const int* __restrict__ tok_pos, int n0, int row_width, int size, int keep,
                                  T* __restrict__ out, size_t total) {
    pdl_trigger();       // the kernel behind may come to rest and wait; it still waits for this one's end
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int n = (int)(i / row_width);
    const Sight s = sight_of(tok_pos[n0 + n], size, keep);
    const int used = (s.n + TV_PART - 1) / TV_PART;        // parts beyond a token's columns hold zeros
    float a = 0.0f;
    for (int z = 0; z < Z && z < used; ++z) a += parts[(size_t)z * part_stride + i];
    out[(size_t)n0 * row_width + i] = from_f32<T>(a);
}

// ---------------------------------------------------------------- prompts: 1. and 3. on the tensor cores
// For steps in which sequences bring many tokens (bfloat16, key and value sizes multiples of
// 16, values of at most 128): a block takes 64 consecutive queries of ONE sequence and one
// head, and walks the cache pages that any of them sees (the pages of the kept first keys,
// then those of the window). A page is a 64-key tile; `mma.sync` m16n8k16 with float32
// accumulators, a warp 16 queries. The scores kernel leaves scale * q . k at each visible
// (query, key) pair's column; the values kernel reads the mixed weights (bfloat16, written
// over the front half of each row by the mix kernel), zero where a key is out of sight, and
// multiplies them with the page's values. Blocks find their sequence and tile from cu_q on the
// device; blocks beyond the step's tiles leave at once. Tokens outside [n0, n0 + n_rows) (the
// rows the scratch matrix holds in this pass) are skipped.
#define TP_Q 64
#define TP_THREADS 128

struct PromptTile {
    int b, tok0, rows, p0, lo_page, hi_page, kept_pages;
};
__device__ __forceinline__ bool prompt_tile(int tile, const int* cu_q, const int* seq_start, int B, int size,
                                            int keep, PromptTile& t) {
    int b = 0;
    for (; b < B; ++b) {
        const int nt = (cu_q[b + 1] - cu_q[b] + TP_Q - 1) / TP_Q;
        if (tile < nt) break;
        tile -= nt;
    }
    if (b == B) return false;
    t.b = b;
    t.tok0 = cu_q[b] + tile * TP_Q;
    t.rows = min(TP_Q, cu_q[b + 1] - t.tok0);
    t.p0 = seq_start[b] + tile * TP_Q;
    const int lo = (size > 0 && t.p0 - size + 1 > 0) ? t.p0 - size + 1 : 0;   // of the tile's first query
    t.lo_page = lo / LUMEN_PAGE;
    t.hi_page = (t.p0 + t.rows - 1) / LUMEN_PAGE;
    t.kept_pages = min((keep + LUMEN_PAGE - 1) / LUMEN_PAGE, t.lo_page);
    return true;
}

// rows x width values of 2 bytes, row-major with `ld` values between rows in global memory,
// into shared memory rows of `pitch` values; rows beyond `rows` are zeroed.
__device__ __forceinline__ void stage_rows(__nv_bfloat16* dst, int pitch, const __nv_bfloat16* src, size_t ld,
                                           int rows, int width) {
    const int chunks = width / 8;
    for (int i = threadIdx.x; i < TP_Q * chunks; i += TP_THREADS) {
        const int r = i / chunks, c = i - r * chunks;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows) v = *reinterpret_cast<const uint4*>(src + (size_t)r * ld + 8 * c);
        *reinterpret_cast<uint4*>(dst + (size_t)r * pitch + 8 * c) = v;
    }
}

// The same for the 64 rows of a cache page, by asynchronous 16-byte copies (one group).
__device__ __forceinline__ void stage_page_async(__nv_bfloat16* dst, int pitch, const __nv_bfloat16* src, int width) {
    const int chunks = width / 8;
    for (int i = threadIdx.x; i < LUMEN_PAGE * chunks; i += TP_THREADS) {
        const int r = i / chunks, c = i - r * chunks;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + (size_t)r * pitch + 8 * c)),
                     "l"(src + (size_t)r * width + 8 * c)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// The pages a tile walks are dealt out over gridDim.z blocks (page k of the walk to block
// k % gridDim.z): the scores of different pages do not meet. While a page is multiplied the
// next one is on its way into the other half of the key buffer.
#define TP_PAGES_A_BLOCK 4
__global__ void __launch_bounds__(TP_THREADS)
talk_scores_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                       const int* __restrict__ table, int table_stride, const int* __restrict__ cu_q,
                       const int* __restrict__ seq_start, int B, float* __restrict__ W, int row_stride, int n0,
                       int n_rows, int H, int G, int d, int size, int keep, float scale) {
    extern __shared__ __align__(16) __nv_bfloat16 sh[];     // queries [64][d + 8], keys 2 x [64][d + 8]
    pdl_trigger();       // the kernel behind may come to rest and wait; it still waits for this one's end
    pdl_wait();
    PromptTile t;
    if (!prompt_tile(blockIdx.x, cu_q, seq_start, B, size, keep, t)) return;
    if (t.tok0 + t.rows <= n0 || t.tok0 >= n0 + n_rows) return;
    const int n_pages = t.kept_pages + t.hi_page - t.lo_page + 1;
    if ((int)blockIdx.z >= n_pages) return;
    const int h = blockIdx.y, g = h / (H / G), pitch = d + 8;
    __nv_bfloat16* Qs = sh;
    __nv_bfloat16* Kbuf = sh + TP_Q * pitch;
    const int* bt = table + (size_t)t.b * table_stride;
    auto page_of = [&](int pi) { return pi < t.kept_pages ? pi : t.lo_page + pi - t.kept_pages; };
    stage_page_async(Kbuf, pitch, kcache + ((size_t)bt[page_of(blockIdx.z)] * G + g) * LUMEN_PAGE * d, d);
    stage_rows(Qs, pitch, q + ((size_t)t.tok0 * H + h) * d, (size_t)H * d, t.rows, d);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int a_row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
    const int b_row = (lane & 7) + 8 * (lane >> 4), b_col = 8 * ((lane >> 3) & 1);
    int buf = 0;
    for (int pi = blockIdx.z; pi < n_pages; pi += gridDim.z, buf ^= 1) {
        const int page_idx = page_of(pi);
        const __nv_bfloat16* Ks = Kbuf + (size_t)buf * LUMEN_PAGE * pitch;
        async_wait_all();
        __syncthreads();             // this page has arrived, and the other half has been read
        if (pi + (int)gridDim.z < n_pages)
            stage_page_async(Kbuf + (size_t)(buf ^ 1) * LUMEN_PAGE * pitch, pitch,
                             kcache + ((size_t)bt[page_of(pi + gridDim.z)] * G + g) * LUMEN_PAGE * d, d);
        float acc[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int k = 0; k < 4; ++k) acc[nt][k] = 0.0f;
        for (int ks = 0; ks < d / 16; ++ks) {
            uint32_t a[4];
            ldsm_x4(a, smem_u32(Qs + (size_t)a_row * pitch + 16 * ks + a_col));
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t bf[4];
                ldsm_x4(bf, smem_u32(Ks + (size_t)(16 * np + b_row) * pitch + 16 * ks + b_col));
                mma_bf16(acc[2 * np], a, bf[0], bf[1]);
                mma_bf16(acc[2 * np + 1], a, bf[2], bf[3]);
            }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int i = warp * 16 + (lane >> 2) + 8 * half;
            const int tok = t.tok0 + i;
            if (i >= t.rows || tok < n0 || tok >= n0 + n_rows) continue;
            const Sight s = sight_of(t.p0 + i, size, keep);
            float* row = W + ((size_t)(tok - n0) * H + h) * row_stride;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int j = page_idx * LUMEN_PAGE + nt * 8 + 2 * (lane & 3) + k;
                    if (j > t.p0 + i || (j < s.lo && j >= s.kept)) continue;
                    row[j < s.kept ? j : s.kept + (j - s.lo)] = acc[nt][2 * half + k] * scale;
                }
        }
    }
}

template <int NT>      // value size / 8
__global__ void __launch_bounds__(TP_THREADS)
talk_values_mma_kernel(const float* __restrict__ W, int row_stride, const __nv_bfloat16* __restrict__ vcache,
                       const int* __restrict__ table, int table_stride, const int* __restrict__ cu_q,
                       const int* __restrict__ seq_start, int B, __nv_bfloat16* __restrict__ out, int n0, int n_rows,
                       int H, int G, int size, int keep) {
    constexpr int dv = NT * 8, vpitch = dv + 8, ppitch = LUMEN_PAGE + 8;
    __shared__ __align__(16) __nv_bfloat16 Ps[TP_Q * ppitch];
    __shared__ __align__(16) __nv_bfloat16 Vbuf[2 * LUMEN_PAGE * vpitch];      // this page's values and the next one's
    pdl_trigger();       // the kernel behind may come to rest and wait; it still waits for this one's end
    pdl_wait();
    PromptTile t;
    if (!prompt_tile(blockIdx.x, cu_q, seq_start, B, size, keep, t)) return;
    if (t.tok0 + t.rows <= n0 || t.tok0 >= n0 + n_rows) return;
    const int h = blockIdx.y, g = h / (H / G);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int* bt = table + (size_t)t.b * table_stride;
    const int a_row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
    const int v_row = (lane & 7) + 8 * ((lane >> 3) & 1), v_col = 8 * (lane >> 4);
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[nt][k] = 0.0f;
    const int n_pages = t.kept_pages + t.hi_page - t.lo_page + 1;
    auto page_of = [&](int pi) { return pi < t.kept_pages ? pi : t.lo_page + pi - t.kept_pages; };
    stage_page_async(Vbuf, vpitch, vcache + ((size_t)bt[page_of(0)] * G + g) * LUMEN_PAGE * dv, dv);
    // A page's weights for the tile's queries: a warp takes its 16 queries one after the other,
    // a lane two neighbouring keys, so a query's 64 weights are one 128-byte read; zero where the
    // key is out of the query's sight.
    unsigned short pw[32];         // raw bfloat16 bits: nothing waits for the loads before the tile is written
    auto fetch_weights = [&](int page_idx) {
#pragma unroll
        for (int rr = 0; rr < 16; ++rr) {
            const int i = warp * 16 + rr, tok = t.tok0 + i;
            const bool live = i < t.rows && tok >= n0 && tok < n0 + n_rows;
            const Sight s = sight_of(t.p0 + (live ? i : 0), size, keep);
            const __nv_bfloat16* row =
                reinterpret_cast<const __nv_bfloat16*>(W + ((size_t)(live ? tok - n0 : 0) * H + h) * row_stride);
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int j = page_idx * LUMEN_PAGE + 2 * lane + k;
                const bool seen = live && j <= t.p0 + i && (j >= s.lo || j < s.kept);
                unsigned short bits = 0;
                if (seen) bits = reinterpret_cast<const unsigned short*>(row)[j < s.kept ? j : s.kept + (j - s.lo)];
                pw[2 * rr + k] = bits;
            }
        }
    };
    fetch_weights(page_of(0));
    for (int pi = 0; pi < n_pages; ++pi) {
        const int page_idx = page_of(pi);
        const __nv_bfloat16* Vs = Vbuf + (size_t)(pi & 1) * LUMEN_PAGE * vpitch;
        __syncthreads();             // the page before has been multiplied
        if (pi + 1 < n_pages)
            stage_page_async(Vbuf + (size_t)((pi + 1) & 1) * LUMEN_PAGE * vpitch, vpitch,
                             vcache + ((size_t)bt[page_of(pi + 1)] * G + g) * LUMEN_PAGE * dv, dv);
        // the page's weights, fetched while the page before was multiplied (below), into their tile
#pragma unroll
        for (int rr = 0; rr < 16; ++rr)
            *reinterpret_cast<uint32_t*>(Ps + (size_t)(warp * 16 + rr) * ppitch + 2 * lane) =
                (uint32_t)pw[2 * rr] | ((uint32_t)pw[2 * rr + 1] << 16);
        // this page's values were asked for a page ago; only the copies just issued may stay in flight
        if (pi + 1 < n_pages) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else async_wait_all();
        __syncthreads();
        if (pi + 1 < n_pages) fetch_weights(page_of(pi + 1));       // in flight while this page is multiplied
#pragma unroll
        for (int ks = 0; ks < LUMEN_PAGE / 16; ++ks) {
            uint32_t a[4];
            ldsm_x4(a, smem_u32(Ps + (size_t)a_row * ppitch + 16 * ks + a_col));
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t bf[4];
                ldsm_x4_t(bf, smem_u32(Vs + (size_t)(16 * ks + v_row) * vpitch + 16 * np + v_col));
                mma_bf16(acc[2 * np], a, bf[0], bf[1]);
                mma_bf16(acc[2 * np + 1], a, bf[2], bf[3]);
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int i = warp * 16 + (lane >> 2) + 8 * half;
        const int tok = t.tok0 + i;
        if (i >= t.rows || tok < n0 || tok >= n0 + n_rows) continue;
        __nv_bfloat16* orow = out + ((size_t)tok * H + h) * dv;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            *reinterpret_cast<uint32_t*>(orow + nt * 8 + 2 * (lane & 3)) = pack_bf16(acc[nt][2 * half], acc[nt][2 * half + 1]);
    }
}

template <int NT>
static void launch_values_mma(dim3 grid, cudaStream_t stream, const float* W, int row_stride, const __nv_bfloat16* vc,
                              const int* table, int table_stride, const int* cu_q, const int* seq_start, int B,
                              __nv_bfloat16* out, int n0, int n_rows, int H, int G, int size, int keep) {
    lumen_launch(talk_values_mma_kernel<NT>, grid, dim3(TP_THREADS), 0, stream, W, row_stride, vc, table, table_stride,
                 cu_q, seq_start, B, out, n0, n_rows, H, G, size, keep);
}

LUMEN_API int lumen_attn_talk_prompt_ok(int H, int G, int d, int dv) {
    return H > 0 && G > 0 && H % G == 0 && H <= TM_MAX_H && d % 16 == 0 && d >= 16 && d <= 256 && dv % 16 == 0 &&
           dv >= 16 && dv <= 128;
}

// The three kernels for a step of prompts. n_tiles bounds the number of (sequence, 64-query)
// tiles (N / 64 + B does for any division of N tokens into B sequences).
LUMEN_API int lumen_attn_talk_prompt(const void* q, const void* kc, const void* vc, const int* table, int table_stride,
                                     const int* cu_q, const int* seq_start, int B, int n_tiles, const int* tok_pos,
                                     const float* talk, void* out, float* W, int N, int rows_per_pass, int row_stride,
                                     int H, int G, int d, int dv, int size, int keep, float scale,
                                     cudaStream_t stream) {
    if (N <= 0) return 0;
    if (!lumen_attn_talk_prompt_ok(H, G, d, dv) || B <= 0 || n_tiles <= 0 || rows_per_pass <= 0 || row_stride <= 0 ||
        size < 0 || keep < 0 || H > 65535)
        return LUMEN_ERR_UNSUPPORTED;
    const size_t smem1 = (size_t)3 * TP_Q * (d + 8) * sizeof(__nv_bfloat16);
    const size_t smem2 = ((size_t)H * H + (size_t)H * TM_THREADS) * sizeof(float);
    if (smem2 > 200 * 1024) return LUMEN_ERR_UNSUPPORTED;
    // pages a tile can walk: its window's (the tile's 64 queries wide), and the kept first keys'
    const int walk = min(row_stride + 2 * LUMEN_PAGE, table_stride * LUMEN_PAGE) / LUMEN_PAGE + 2;
    const dim3 grid1(n_tiles, H, max(1, min(64, (walk + TP_PAGES_A_BLOCK - 1) / TP_PAGES_A_BLOCK)));
    if (smem1 > 40 * 1024)
        cudaFuncSetAttribute(talk_scores_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    const dim3 grid(n_tiles, H);
    for (int n0 = 0; n0 < N; n0 += rows_per_pass) {
        const int rows = min(rows_per_pass, N - n0);
        lumen_launch(talk_scores_mma_kernel, grid1, dim3(TP_THREADS), smem1, stream, (const __nv_bfloat16*)q,
                     (const __nv_bfloat16*)kc, table, table_stride, cu_q, seq_start, B, W, row_stride, n0, rows, H, G, d,
                     size, keep, scale);
        launch_mix(rows, stream, W, row_stride, tok_pos, n0, talk, H, size, keep);
#define LUMEN_TALK_VALUES(NT_)                                                                                        \
    case NT_:                                                                                                         \
        launch_values_mma<NT_>(grid, stream, (const float*)W, row_stride, (const __nv_bfloat16*)vc, table,            \
                               table_stride, cu_q, seq_start, B, (__nv_bfloat16*)out, n0, rows, H, G, size, keep);    \
        break;
        switch (dv / 8) {
            LUMEN_TALK_VALUES(2) LUMEN_TALK_VALUES(4) LUMEN_TALK_VALUES(6) LUMEN_TALK_VALUES(8) LUMEN_TALK_VALUES(10)
            LUMEN_TALK_VALUES(12) LUMEN_TALK_VALUES(14) LUMEN_TALK_VALUES(16)
            default: return LUMEN_ERR_UNSUPPORTED;
        }
#undef LUMEN_TALK_VALUES
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

// ---------------------------------------------------------------- host side
// q [N, H, d], out [N, H, dv]; scratch: W (scores) float32 [rows, H, row_stride] and stats float32
// [rows, H, chunks of 64 columns, 2] with rows >= min(N, rows_per_pass); parts: float32 [Z, rows, H, dv] when row_stride > TV_PART (Z parts), else null.
template <typename T>
static int attn_talk_run(const T* q, const T* kc, const T* vc, const int* table, int table_stride, const int* tok_seq,
                         const int* tok_pos, const float* talk, T* out, float* W, float* stats,
                         float* parts, int N,
                         int rows_per_pass, int row_stride, int H, int G, int d, int dv, int size, int keep,
                         float scale, int k_layout, int v_layout, cudaStream_t stream) {
    // blocks a kv head's heads are dealt out over: equal shares of at most 16 heads whose sums and
    // mixed weights fit the values kernel's shared memory
    const int E = (dv <= 128 && dv % 4 == 0) ? 4 : 8;
    auto values_smem = [&](int per_) {
        return ((size_t)(TV_THREADS / 32) * per_ * 32 * E + (size_t)2 * per_ * TV_PART + (size_t)per_ * H + 2 * H) * sizeof(float);
    };
    int hsplit = 1;
    while ((H / G) % hsplit || (H / G) / hsplit > TS_MAX_PER || (values_smem((H / G) / hsplit) > 48 * 1024 && hsplit < H / G))
        ++hsplit;
    const int per = H / G / hsplit;
    const int chunks = (row_stride + TS_COLS - 1) / TS_COLS;
    const int Z = (row_stride + TV_PART - 1) / TV_PART;
    const size_t smem1 = (size_t)per * (d + TS_COLS) * sizeof(float);
    const size_t smem3 = values_smem(per);
    if (smem1 > 160 * 1024 || smem3 > 48 * 1024) return LUMEN_ERR_UNSUPPORTED;
    if (smem1 > 40 * 1024)
        cudaFuncSetAttribute(talk_scores_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    for (int n0 = 0; n0 < N; n0 += rows_per_pass) {
        const int rows = min(rows_per_pass, N - n0);
        lumen_launch(talk_scores_kernel<T>, dim3(rows, G * hsplit, chunks), dim3(TS_THREADS), smem1, stream, q, kc, table,
                     table_stride, tok_seq, tok_pos, W, stats, row_stride, n0, H, G, d, size, keep, scale, k_layout, hsplit);
        if (E == 4)
            launch_values<T, 4>(per, dim3(rows, G * hsplit, Z), smem3, stream, (const float*)W, (const float*)stats,
                                chunks, talk, row_stride, vc, table,
                                table_stride, tok_seq, tok_pos, out, Z > 1 ? parts : (float*)nullptr, n0, rows, H, G, dv,
                                size, keep, v_layout, hsplit);
        else
            launch_values<T, 8>(per, dim3(rows, G * hsplit, Z), smem3, stream, (const float*)W, (const float*)stats,
                                chunks, talk, row_stride, vc, table,
                                table_stride, tok_seq, tok_pos, out, Z > 1 ? parts : (float*)nullptr, n0, rows, H, G, dv,
                                size, keep, v_layout, hsplit);
        if (Z > 1) {
            const size_t total = (size_t)rows * H * dv;
            lumen_launch(talk_parts_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                         (const float*)parts, Z, total, tok_pos, n0, H * dv, size, keep, out, total);
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

LUMEN_API int lumen_attn_talk(const void* q, const void* kc, const void* vc, const int* table, int table_stride,
                              const int* tok_seq, const int* tok_pos, const float* talk, void* out, float* W,
                              float* stats, float* parts, int is_bf16, int N, int rows_per_pass, int row_stride, int H, int G, int d,
                              int dv, int size, int keep, float scale, int k_layout, int v_layout,
                              cudaStream_t stream) {
    if (N <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || H > TM_MAX_H || d <= 0 || dv <= 0 || dv > 256 ||
        rows_per_pass <= 0 || row_stride <= 0 || size < 0 || keep < 0 || H > 65535)
        return LUMEN_ERR_UNSUPPORTED;
    if ((row_stride + TS_COLS - 1) / TS_COLS > 65535) return LUMEN_ERR_UNSUPPORTED;
    if ((k_layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || d % 64)) || (v_layout == LUMEN_LAYOUT_SW128 && (!is_bf16 || dv % 64)))
        return LUMEN_ERR_UNSUPPORTED;
    if ((row_stride > TV_PART && !parts) || !W || !stats) return LUMEN_ERR_BAD_ARGUMENT;
    if (is_bf16)
        return attn_talk_run<__nv_bfloat16>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                                            table, table_stride, tok_seq, tok_pos, talk, (__nv_bfloat16*)out, W, stats, parts, N,
                                            rows_per_pass, row_stride, H, G, d, dv, size, keep, scale, k_layout,
                                            v_layout, stream);
    return attn_talk_run<float>((const float*)q, (const float*)kc, (const float*)vc, table, table_stride, tok_seq,
                                tok_pos, talk, (float*)out, W, stats, parts, N, rows_per_pass, row_stride, H, G, d, dv, size,
                                keep, scale, k_layout, v_layout, stream);
}
