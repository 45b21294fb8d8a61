// The gated delta rule, token by token, over the rows of a step.
//
// A head keeps a memory S [d, e] (d: key size, e: value size). With a decay g in (0, 1), a step size
// beta in (0, 1), a unit key k, a unit query q (times d^-1/2) and a value v, a row does
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// so the read-out sees the row's own write. q, k (of `kv_heads` heads, shared by heads / kv_heads heads
// each) and v come from a stacked product [rows, row_width] through a short causal convolution over
// time, one filter a channel (`taps` weights, the last for the row itself, zeros before a request's
// first row), and silu. g = exp(-exp(A_log) softplus(a + dt_bias)) and beta = sigmoid(b) come from two
// more columns a head. The memory and the last taps - 1 inputs of every channel live in a slot of a
// float32 state table, one slot a request, and are carried from a request's last row in this step to
// its first row in the next. Everything here is 32-bit; only the projections may come in bfloat16.
//
// Three kernels. `delta_prep_kernel`, a block a row: convolution and silu of every channel (rows before
// the step come from the slot's history), unit norms of q and k per head, q.k per kv head, decay and
// step size per head, all left in 32-bit scratch. `delta_history_kernel`, a thread a channel of a
// request: the slot's history becomes the last taps - 1 inputs. `delta_scan_kernel`: one block = one
// request of the step x one head x 4, 8 or 16 value components, a warp one, two or four of them, lane l the memory's
// rows j = l, l + 32, ... of those columns in registers. Written with the decayed memory M = g S of a row:
// a = M.k and b = M.q of a warp's columns are reduced together (5, 6 or 9 shuffles a row), u = beta (v - a),
// o = b + u (k.q), S = M + k u. The rows' inputs come into shared memory a chunk of rows at a time by
// asynchronous copies, the next chunk while this one is walked. A
// column of a head's memory lies together in the state table, so a warp reads and writes whole lines.
#include "common.cuh"

namespace kb {

typedef __nv_bfloat16 bf16;

constexpr int DC = 4;                  // value components (warps) a block of the scan
constexpr int DELTA_MAX_TAPS = 8;
constexpr int DELTA_R = 8;             // memory rows a lane can hold: d <= 32 * DELTA_R

struct DeltaParams {
    int row_width;              // columns of the stacked product
    int q_off, k_off, v_off, b_off, a_off;
    const float* conv;          // [channels, taps]: q's channels, then k's, then v's
    const float* a_log;         // [heads]
    const float* dt_bias;       // [heads]
    float* state;               // [slots, state_floats]: history [taps - 1, channels], then S [heads, e, d]
    long long state_floats;
    const int* row_entry;       // [rows]
    const int* entry_start;     // [entries]
    const int* entry_end;
    const int* slots;           // [entries]; slot 0 belongs to rows that are no token's
    int n_slots, entries, rows, heads, kv_heads, d, e, taps;
    float q_scale, unit_eps;
    float* qn;                  // [rows, kv_heads, d] scratch
    float* kn;                  // [rows, kv_heads, d]
    float* vn;                  // [rows, heads, e]
    float* scal;                // [rows, heads, 2] decay, step size;
    float* kq;                  // [rows, kv_heads]
    float* out;                 // [rows, heads, e]
};

__device__ __forceinline__ float delta_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float delta_silu(float x) { return x / (1.f + expf(-x)); }

template <typename TS>
__global__ void __launch_bounds__(1024)
delta_prep_kernel(const Src<TS> src, const DeltaParams p) {
    extern __shared__ float act[];                              // [channels]
    const int r = blockIdx.x;
    const int nq = p.kv_heads * p.d, nv = p.heads * p.e;
    const int channels = 2 * nq + nv;
    const int entry = p.row_entry[r];
    int r0 = r, slot = 0;
    if (entry >= 0 && entry < p.entries) {
        r0 = p.entry_start[entry];
        slot = p.slots[entry];
    }
    const bool kept = slot > 0 && slot < p.n_slots;
    const float* hist = p.state + (size_t)(kept ? slot : 0) * p.state_floats;
    const int taps = p.taps;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        const int col = c < nq ? p.q_off + c : (c < 2 * nq ? p.k_off + (c - nq) : p.v_off + (c - 2 * nq));
        float y = 0.f;
        for (int j = 0; j < taps; ++j) {                        // the input j rows back
            const int t = r - j;
            float x;
            if (t >= r0) x = src.at((size_t)t * p.row_width + col);
            else if (kept) x = hist[(size_t)(taps - 1 + (t - r0)) * channels + c];     // t - r0 in [-(taps-1), -1]
            else x = 0.f;
            y = fmaf(p.conv[(size_t)c * taps + (taps - 1 - j)], x, y);
        }
        act[c] = delta_silu(y);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    // unit vectors per kv head, and q.k
    for (int h = warp; h < p.kv_heads; h += warps) {
        float sq = 0.f, sk = 0.f, qk = 0.f;
        for (int i = lane; i < p.d; i += 32) {
            const float q = act[h * p.d + i], k = act[nq + h * p.d + i];
            sq = fmaf(q, q, sq);
            sk = fmaf(k, k, sk);
            qk = fmaf(q, k, qk);
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        qk = warp_sum(qk);
        const float iq = p.q_scale / sqrtf(sq + p.unit_eps), ik = 1.f / sqrtf(sk + p.unit_eps);
        for (int i = lane; i < p.d; i += 32) {
            p.qn[((size_t)r * p.kv_heads + h) * p.d + i] = act[h * p.d + i] * iq;
            p.kn[((size_t)r * p.kv_heads + h) * p.d + i] = act[nq + h * p.d + i] * ik;
        }
        if (lane == 0) p.kq[(size_t)r * p.kv_heads + h] = qk * iq * ik;
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) p.vn[(size_t)r * nv + i] = act[2 * nq + i];
    for (int h = threadIdx.x; h < p.heads; h += blockDim.x) {
        const float a = src.at((size_t)r * p.row_width + p.a_off + h) + p.dt_bias[h];
        const float b = src.at((size_t)r * p.row_width + p.b_off + h);
        p.scal[((size_t)r * p.heads + h) * 2] = expf(-expf(p.a_log[h]) * delta_softplus(a));
        p.scal[((size_t)r * p.heads + h) * 2 + 1] = 1.f / (1.f + expf(-b));
    }
}

// history <- the last taps - 1 inputs of (history, this step's rows), per channel of a request.
template <typename TS>
__global__ void delta_history_kernel(const Src<TS> src, const DeltaParams p) {
    const int entry = blockIdx.y;
    const int nq = p.kv_heads * p.d, nv = p.heads * p.e;
    const int channels = 2 * nq + nv;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int r0 = p.entry_start[entry], r1 = p.entry_end[entry];
    const int slot = p.slots[entry];
    if (r1 <= r0 || slot <= 0 || slot >= p.n_slots) return;
    const int keep = p.taps - 1;
    if (keep <= 0) return;
    float* hist = p.state + (size_t)slot * p.state_floats;
    const int col = c < nq ? p.q_off + c : (c < 2 * nq ? p.k_off + (c - nq) : p.v_off + (c - 2 * nq));
    const int n = r1 - r0;
    float fresh[DELTA_MAX_TAPS];
#pragma unroll
    for (int i = 0; i < DELTA_MAX_TAPS; ++i) {
        fresh[i] = 0.f;
        if (i < keep) {
            const int t = n - keep + i;                         // the input at this place, counted from the step's first row
            fresh[i] = t >= 0 ? src.at((size_t)(r0 + t) * p.row_width + col) : hist[(size_t)(keep + t) * channels + c];
        }
    }
#pragma unroll
    for (int i = 0; i < DELTA_MAX_TAPS; ++i)
        if (i < keep) hist[(size_t)i * channels + c] = fresh[i];
}

__device__ __forceinline__ void delta_copy4(float* dst, const float* src) {
    const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d32), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_copy16(float* dst, const float* src) {
    const uint32_t d32 = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d32), "l"(src) : "memory");
}

// R: memory rows a lane holds (d <= 32 R); CH: rows of the step staged at a time. The rows' inputs (k, q, the block's
// values, decay, step size, q.k) come into shared memory a chunk at a time by asynchronous copies, the next chunk
// while this one is walked: a row's step then waits for shared memory only. A warp holds DW columns of the memory,
// so k and q are read once for all of them and the 2 DW dot products of a row are reduced together: each round of
// shuffles halves the number of sums a lane carries (9 shuffles for 8 sums instead of 40).
// DW (1, 2 or 4): columns a warp; the launcher takes the most that still leaves the GPU enough warps.
template <int R, int CH, int DW>
__global__ void __launch_bounds__(DC * 32)
delta_scan_kernel(const DeltaParams p) {
    constexpr int DCOLS = DC * DW;                              // columns a block
    constexpr int SHIFT = DW == 4 ? 2 : (DW == 2 ? 3 : 4);     // the sum of column c ends in lane c << SHIFT (M.k) and 16 + (c << SHIFT) (M.q)
    extern __shared__ __align__(16) float staged[];             // [2][CH][rowf]
    const int entry = blockIdx.x, head = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c0 = blockIdx.z * DCOLS + warp * DW;              // this warp's first column
    const int r0 = p.entry_start[entry], r1 = p.entry_end[entry];
    if (r1 <= r0) return;
    const int slot = p.slots[entry];
    const int d = p.d, e = p.e;
    if (slot <= 0 || slot >= p.n_slots) {                       // rows of no request: zeros, no state
        if (lane < DW && c0 + lane < e)
            for (int r = r0; r < r1; ++r) p.out[((size_t)r * p.heads + head) * e + c0 + lane] = 0.f;
        return;
    }
    const int nq = p.kv_heads * d, nv = p.heads * e;
    const int kvh = head / (p.heads / p.kv_heads);
    float* st = p.state + (size_t)slot * p.state_floats + (size_t)(p.taps - 1) * (2 * nq + nv) + (size_t)head * e * d;
    float S[DW][R];
#pragma unroll
    for (int ci = 0; ci < DW; ++ci)
#pragma unroll
        for (int i = 0; i < R; ++i) S[ci][i] = (c0 + ci < e && lane + 32 * i < d) ? st[(size_t)(c0 + ci) * d + lane + 32 * i] : 0.f;

    constexpr int DP = R * 32;                                  // k and q padded to the lanes' rows, zeros beyond d
    constexpr int tail = 2 * DP;                                // v [DCOLS] | decay | step size | q.k | padding
    constexpr int rowf = 2 * DP + DCOLS + 8;
    const bool wide = d % 4 == 0 && (((uintptr_t)p.kn | (uintptr_t)p.qn) & 15) == 0;
    auto stage = [&](int chunk, int buf) {
        const int rbase = r0 + chunk * CH;
        const int nr = min(CH, r1 - rbase);
        float* base = staged + (size_t)buf * CH * rowf;
        for (int t = warp; t < nr; t += DC) {                   // a warp a row in turn
            float* row = base + (size_t)t * rowf;
            const float* kp = p.kn + ((size_t)(rbase + t) * p.kv_heads + kvh) * d;
            const float* qp = p.qn + ((size_t)(rbase + t) * p.kv_heads + kvh) * d;
            if (wide) {
                for (int x = lane * 4; x < d; x += 128) {
                    delta_copy16(row + x, kp + x);
                    delta_copy16(row + DP + x, qp + x);
                }
            } else {
                for (int x = lane; x < d; x += 32) {
                    delta_copy4(row + x, kp + x);
                    delta_copy4(row + DP + x, qp + x);
                }
            }
        }
        for (int idx = tid; idx < nr * (DCOLS + 3); idx += DC * 32) {
            const int t = idx / (DCOLS + 3), x = idx - t * (DCOLS + 3);
            float* dst = base + (size_t)t * rowf + tail + x;
            const size_t r = (size_t)(rbase + t);
            if (x < DCOLS) {
                const int cc = blockIdx.z * DCOLS + x;
                if (cc < e) delta_copy4(dst, p.vn + (r * p.heads + head) * e + cc);
                else *dst = 0.f;
            } else if (x < DCOLS + 2) {
                delta_copy4(dst, p.scal + (r * p.heads + head) * 2 + (x - DCOLS));
            } else {
                delta_copy4(dst, p.kq + r * p.kv_heads + kvh);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (d < DP) {                                               // the padding of k and q, once: no copy ever writes it
        for (int idx = tid; idx < 2 * CH * 2 * (DP - d); idx += DC * 32) {
            const int t = idx / (2 * (DP - d)), x = idx - t * 2 * (DP - d);
            staged[(size_t)t * rowf + (x < DP - d ? d + x : DP + d + (x - (DP - d)))] = 0.f;
        }
    }
    const bool hi16 = lane & 16, hi8 = lane & 8, hi4 = lane & 4;
    const int mine = (lane & 15) >> SHIFT;                      // the column whose sum this lane ends up with
    const int chunks = (r1 - r0 + CH - 1) / CH;
    stage(0, 0);
    for (int ch = 0; ch < chunks; ++ch) {
        if (ch + 1 < chunks) {
            stage(ch + 1, (ch + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int rbase = r0 + ch * CH;
        const int nr = min(CH, r1 - rbase);
        const float* rows = staged + (size_t)(ch & 1) * CH * rowf;
        for (int t = 0; t < nr; ++t) {
            const float* in = rows + (size_t)t * rowf;
            const float g = in[tail + DCOLS], beta = in[tail + DCOLS + 1], kq = in[tail + DCOLS + 2];
            float k[R], q[R];
#pragma unroll
            for (int i = 0; i < R; ++i) {
                k[i] = in[lane + 32 * i];
                q[i] = in[DP + lane + 32 * i];
            }
            float x[2 * DW];                                    // a lane's share of M.k for each column, then of M.q
#pragma unroll
            for (int ci = 0; ci < DW; ++ci) {
                float a = 0.f, b = 0.f;
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    S[ci][i] *= g;
                    a = fmaf(S[ci][i], k[i], a);
                    b = fmaf(S[ci][i], q[i], b);
                }
                x[ci] = a;
                x[DW + ci] = b;
            }
            // 2 DW sums over 32 lanes: each round a lane hands half of what it carries to its partner
            float w;
            if constexpr (DW == 4) {
                float y[4], z[2];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float send = hi16 ? x[i] : x[i + 4], keep = hi16 ? x[i + 4] : x[i];
                    y[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float send = hi8 ? y[i] : y[i + 2], keep = hi8 ? y[i + 2] : y[i];
                    z[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                }
                w = (hi4 ? z[1] : z[0]) + __shfl_xor_sync(0xffffffffu, hi4 ? z[0] : z[1], 4);
            } else if constexpr (DW == 2) {
                float y[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float send = hi16 ? x[i] : x[i + 2], keep = hi16 ? x[i + 2] : x[i];
                    y[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
                }
                w = (hi8 ? y[1] : y[0]) + __shfl_xor_sync(0xffffffffu, hi8 ? y[0] : y[1], 8);
                w += __shfl_xor_sync(0xffffffffu, w, 4);
            } else {
                w = (hi16 ? x[1] : x[0]) + __shfl_xor_sync(0xffffffffu, hi16 ? x[0] : x[1], 16);
                w += __shfl_xor_sync(0xffffffffu, w, 8);
                w += __shfl_xor_sync(0xffffffffu, w, 4);
            }
            w += __shfl_xor_sync(0xffffffffu, w, 2);
            w += __shfl_xor_sync(0xffffffffu, w, 1);
            // lanes 0..15 now hold M.k of column (lane & 15) >> SHIFT, lanes 16..31 M.q of that column
            float u[DW];
#pragma unroll
            for (int ci = 0; ci < DW; ++ci) {
                const float a = __shfl_sync(0xffffffffu, w, ci << SHIFT);
                u[ci] = beta * (in[tail + warp * DW + ci] - a);
#pragma unroll
                for (int i = 0; i < R; ++i) S[ci][i] = fmaf(k[i], u[ci], S[ci][i]);
            }
            if (hi16 && (lane & ((1 << SHIFT) - 1)) == 0 && c0 + mine < e) {
                float um = u[0];
#pragma unroll
                for (int ci = 1; ci < DW; ++ci) um = mine == ci ? u[ci] : um;
                p.out[((size_t)(rbase + t) * p.heads + head) * e + c0 + mine] = fmaf(um, kq, w);
            }
        }
        __syncthreads();                                        // the chunk's buffer may be written again
    }
#pragma unroll
    for (int ci = 0; ci < DW; ++ci)
#pragma unroll
        for (int i = 0; i < R; ++i)
            if (c0 + ci < e && lane + 32 * i < d) st[(size_t)(c0 + ci) * d + lane + 32 * i] = S[ci][i];
}

}  // namespace kb

using namespace kb;

// 0: the launcher chooses how many columns of the memory a warp of the scan holds; 1, 2 or 4: that many (for tests and measurements).
static int g_delta_columns = 0;
extern "C" void kb_delta_columns_per_warp(int n) { g_delta_columns = (n == 1 || n == 2 || n == 4) ? n : 0; }

// Floats a request keeps between steps: the convolutions' history, then every head's memory.
extern "C" long long kb_delta_state_floats(int heads, int kv_heads, int d, int e, int taps) {
    return (long long)(taps - 1) * (2ll * kv_heads * d + (long long)heads * e) + (long long)heads * d * e;
}

// Floats of scratch for a step of `rows` rows: unit queries and keys, values, (decay, step size), q.k.
extern "C" long long kb_delta_scratch_floats(int rows, int heads, int kv_heads, int d, int e) {
    return (long long)rows * (2ll * kv_heads * d + (long long)heads * e + 2ll * heads + kv_heads);
}

extern "C" int kb_delta_scan(float* out, float* scratch, const void* src, int in_dt, int splits, long long split_stride, int row_width,
                             int q_off, int k_off, int v_off, int b_off, int a_off, const float* conv, const float* a_log,
                             const float* dt_bias, float* state, int n_slots, long long state_floats, const int* row_entry,
                             const int* entry_start, const int* entry_end, const int* slots, int entries, int rows, int heads,
                             int kv_heads, int d, int e, int taps, float q_scale, float unit_eps, void* stream) {
    KB_REQUIRE(entries >= 0 && rows >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && d > 0 && e > 0,
               "delta: entries %d, rows %d, heads %d over %d, sizes %d / %d", entries, rows, heads, kv_heads, d, e);
    KB_REQUIRE(d <= 32 * DELTA_R, "delta: a key size of %d is more than the kernel's %d", d, 32 * DELTA_R);
    KB_REQUIRE(taps >= 1 && taps <= DELTA_MAX_TAPS, "delta: a convolution of %d taps (1 to %d)", taps, DELTA_MAX_TAPS);
    const long long nq = (long long)kv_heads * d, nv = (long long)heads * e;
    KB_REQUIRE(row_width > 0 && q_off >= 0 && q_off + nq <= row_width && k_off >= 0 && k_off + nq <= row_width && v_off >= 0 &&
                   v_off + nv <= row_width && b_off >= 0 && b_off + heads <= row_width && a_off >= 0 && a_off + heads <= row_width,
               "delta: columns q %d, k %d, v %d, b %d, a %d do not fit a row of %d", q_off, k_off, v_off, b_off, a_off, row_width);
    KB_REQUIRE(splits >= 1 && (splits == 1 || split_stride >= (long long)rows * row_width), "delta: %d slices %lld apart", splits, split_stride);
    KB_REQUIRE(state_floats == kb_delta_state_floats(heads, kv_heads, d, e, taps), "delta: a state of %lld floats, expected %lld",
               state_floats, kb_delta_state_floats(heads, kv_heads, d, e, taps));
    KB_REQUIRE(n_slots >= 1 && state && scratch && out && conv && a_log && dt_bias && row_entry && entry_start && entry_end && slots,
               "delta: state, scratch, weights or ranges are missing");
    if (entries == 0 || rows == 0) return 0;
    const long long channels = 2 * nq + nv;
    KB_REQUIRE(channels * 4 <= 200 * 1024, "delta: %lld channels do not fit the shared memory of a block", channels);
    KB_REQUIRE(heads <= 65535 && entries <= 65535 && (e + DC * 4 - 1) / (DC * 4) <= 65535, "delta: too many heads, requests or value components for one launch");
    DeltaParams p;
    p.row_width = row_width; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.b_off = b_off; p.a_off = a_off;
    p.conv = conv; p.a_log = a_log; p.dt_bias = dt_bias; p.state = state; p.state_floats = state_floats; p.row_entry = row_entry;
    p.entry_start = entry_start; p.entry_end = entry_end; p.slots = slots; p.n_slots = n_slots; p.entries = entries; p.rows = rows;
    p.heads = heads; p.kv_heads = kv_heads; p.d = d; p.e = e; p.taps = taps; p.q_scale = q_scale; p.unit_eps = unit_eps;
    p.qn = scratch;
    p.kn = p.qn + (size_t)rows * nq;
    p.vn = p.kn + (size_t)rows * nq;
    p.scal = p.vn + (size_t)rows * nv;
    p.kq = p.scal + (size_t)rows * heads * 2;
    p.out = out;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)channels * sizeof(float);
#define KB_DELTA_PREP(TS)                                                                                                  \
    do {                                                                                                                   \
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prep_kernel<TS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        delta_prep_kernel<TS><<<rows, rows <= DEPENDENT_ROWS ? 1024 : 256, smem, s>>>(Src<TS>{(const TS*)src, splits, (size_t)split_stride}, p); /* few rows: a channel or two a thread */ \
        if (int err = check_launch("delta prep")) return err;                                                              \
        if (taps > 1) {                                                                                                    \
            delta_history_kernel<TS><<<dim3((unsigned)((channels + 127) / 128), entries), 128, 0, s>>>(                     \
                Src<TS>{(const TS*)src, splits, (size_t)split_stride}, p);                                                 \
            if (int err = check_launch("delta history")) return err;                                                       \
        }                                                                                                                  \
    } while (0)
    if (in_dt == KB_DT_F32) KB_DELTA_PREP(float);
    else if (in_dt == KB_DT_BF16) KB_DELTA_PREP(bf16);
    else return fail("delta: dtype code %d is not known", in_dt);
#undef KB_DELTA_PREP
    // columns a warp: the most that still gives the GPU about eight warps a multiprocessor (a prompt of one request has
    // heads x value components warps at one column each; a batch of requests has many times that)
    int sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const long long columns = (long long)entries * heads * e;
    const int dw = g_delta_columns ? g_delta_columns : (columns / 4 >= 16ll * sms ? 4 : (columns / 2 >= 8ll * sms ? 2 : 1));
    KB_REQUIRE((e + DC * dw - 1) / (DC * dw) <= 65535, "delta: too many value components for one launch");
    dim3 grid(entries, heads, (e + DC * dw - 1) / (DC * dw));
    const int need = (d + 31) / 32;
#define KB_DELTA_SCAN(R, CH, W) delta_scan_kernel<R, CH, W><<<grid, DC * 32, (size_t)2 * CH * (2 * R * 32 + DC * W + 8) * sizeof(float), s>>>(p)
#define KB_DELTA_SCAN_W(R, CH)            \
    do {                                  \
        if (dw == 4) KB_DELTA_SCAN(R, CH, 4);      \
        else if (dw == 2) KB_DELTA_SCAN(R, CH, 2); \
        else KB_DELTA_SCAN(R, CH, 1);     \
    } while (0)
    if (need <= 1) KB_DELTA_SCAN_W(1, 16);
    else if (need <= 2) KB_DELTA_SCAN_W(2, 16);
    else if (need <= 4) KB_DELTA_SCAN_W(4, 16);
    else KB_DELTA_SCAN_W(DELTA_R, 8);
#undef KB_DELTA_SCAN_W
#undef KB_DELTA_SCAN
    return check_launch("delta scan");
}
