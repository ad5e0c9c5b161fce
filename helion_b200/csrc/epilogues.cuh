// Epilogue functors shared by the tcgen05 GEMM core and the CUDA-core (SIMT) GEMM core.
//
// Both cores hand an accumulator tile to the functor the same way: one thread owns one row of the
// tile and receives it 32 consecutive fp32 columns at a time.
//   begin(state, params, tile)            once per tile, before any column arrives
//   chunk(state, params, tile, col0, v)   v[j] = D[row, col0 + j], col0 relative to the tile
//   end(state, params, tile)              once per tile, after the last chunk
// Row reductions are therefore thread-local: no shuffles, no shared memory.
#pragma once

#include <type_traits>

#include "gemm_tc.cuh"

namespace lce {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <class T> struct Cvt;
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};
template <> struct Cvt<float> {
    static __device__ __forceinline__ float to_f(float x) { return x; }
    static __device__ __forceinline__ float from_f(float x) { return x; }
};

__device__ __forceinline__ long long load_target(const void* tgt, int is_i64, long long i) {
    return is_i64 ? static_cast<const long long*>(tgt)[i]
                  : static_cast<long long>(static_cast<const int*>(tgt)[i]);
}

// Stores 32 consecutive values of one row. Vectorised (16-byte) when the whole chunk is in
// bounds and the destination is 16-byte aligned; element-wise on the ragged edge.
template <class T>
__device__ __forceinline__ void store_row32(T* dst, const float (&v)[32], int ncols_valid) {
    constexpr int kPerVec = 16 / sizeof(T);
    if (ncols_valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < 32 / kPerVec; ++i) {
            alignas(16) T tmp[kPerVec];
#pragma unroll
            for (int j = 0; j < kPerVec; ++j) tmp[j] = Cvt<T>::from_f(v[i * kPerVec + j]);
            *reinterpret_cast<uint4*>(dst + i * kPerVec) = *reinterpret_cast<const uint4*>(tmp);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < ncols_valid) dst[j] = Cvt<T>::from_f(v[j]);
    }
}

// Line-wide stores of 16-bit results. A thread owns one row and receives it 32 columns at a time; stored
// directly, every store instruction touches 32 rows with 16 bytes each - 32 partial-sector requests, which
// is what bounds a GEMM with a short contraction (the output is large, the main loop short). Here the warp
// parks two consecutive chunks (64 columns = 128 bytes per row) in its shared-memory area and then writes
// whole 128-byte lines: 8 lanes per row, 4 rows per store instruction.
// Area layout: [32 rows][8 pieces of 16 bytes], the piece index XORed with the row's low three bits, so the
// row-wise deposit and the line-wise pick-up are both free of bank conflicts.
// All 32 lanes call this for every chunk of the tile, in column order; half = (col0 / 32) & 1.
//   out_blk     address of (first row of this warp, first column of the 64-column block), 16-byte aligned
//   ld          row pitch in elements, a multiple of 8
//   rows_valid  how many of the warp's 32 rows exist (<= 0: none)
//   cols_valid  how many of the block's 64 columns exist (<= 0: none)
template <class T>
__device__ __forceinline__ void store_block64(float* stage, int lane, int half, const float (&v)[32], T* out_blk,
                                              long long ld, int rows_valid, int cols_valid) {
    static_assert(sizeof(T) == 2, "16-bit outputs only");
    uint4* sm = reinterpret_cast<uint4*>(stage);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        alignas(16) T tmp[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) tmp[j] = Cvt<T>::from_f(v[i * 8 + j]);
        sm[lane * 8 + ((half * 4 + i) ^ (lane & 7))] = *reinterpret_cast<const uint4*>(tmp);
    }
    if (half == 0) return;
    __syncwarp();
    const int piece = lane & 7;
    const int left = cols_valid - piece * 8;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + (lane >> 3);
        const uint4 val = sm[r * 8 + (piece ^ (r & 7))];
        if (r < rows_valid && left > 0) {
            T* dst = out_blk + static_cast<long long>(r) * ld + piece * 8;
            if (left >= 8) {
                *reinterpret_cast<uint4*>(dst) = val;
            } else {
                const T* e = reinterpret_cast<const T*>(&val);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < left) dst[j] = e[j];
            }
        }
    }
    __syncwarp();  // the area is free again
}

// ---------------------------------------------------------------------------------------------
// Forward: per (vocab tile, row) partial softmax statistics.
//   partial[(n_tile*3 + 0) * row_stride + row] = max_j z[row, j]
//   partial[(n_tile*3 + 1) * row_stride + row] = sum_j exp(z[row, j] - max)
//   partial[(n_tile*3 + 2) * row_stride + row] = z[row, target] if the target falls in this tile
//                                                else -inf
// Columns at or beyond `vocab` (zero-filled by TMA) are masked to -inf. The same three numbers
// per block are what the reference's partial-forward kernel emits
// (tritium/ops/cross_entropy.py:235-248).
// ---------------------------------------------------------------------------------------------
struct EpiStats {
    // The CTA that finishes last can merge the partial statistics and write logsumexp and loss itself
    // (finish(), small batches of an unsharded vocabulary only): the forward is then ONE launch.
    static constexpr bool kHasFinish = true;
    struct Params {
        const void* tgt;
        int tgt_i64;
        int rows;               // valid rows
        int vocab;              // valid columns (local shard width)
        long long vocab_start;  // global index of local column 0
        float* partial;
        long long row_stride;
        // finish(): outputs of the fused tail (used only when the launch is given a completion counter)
        float* fin_lse = nullptr;          // [rows]
        float* fin_loss = nullptr;         // () for mean / sum, [rows] for none
        float* fin_valid_count = nullptr;  // optional
        int fin_reduction = 1;
        long long fin_ignore_index = -100;
        int fin_n_tiles = 0;
    };
    static __device__ void finish(const Params& p);
    struct State {
        float m, s, t;
        int tcol;  // target column relative to the tile, or -1
        int row;
    };
    static __device__ __forceinline__ void begin(State& st, const Params& p, const TileCtx& tc) {
        st.row = tc.m_tile * kBM + tc.row_in_tile;
        st.m = -INFINITY;
        st.s = 0.f;
        st.t = -INFINITY;
        st.tcol = -1;
        if (st.row < p.rows) {
            const long long rel = load_target(p.tgt, p.tgt_i64, st.row) - p.vocab_start -
                                  static_cast<long long>(tc.n_tile) * tc.bn;
            if (rel >= 0 && rel < tc.bn && rel + static_cast<long long>(tc.n_tile) * tc.bn < p.vocab)
                st.tcol = static_cast<int>(rel);
        }
    }
    static __device__ __forceinline__ void chunk(State& st, const Params& p, const TileCtx& tc,
                                                 int col0, float (&v)[32]) {
        const int gcol0 = tc.n_tile * tc.bn + col0;
        if (gcol0 >= p.vocab) return;
        if (gcol0 + 32 > p.vocab) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (gcol0 + j >= p.vocab) v[j] = -INFINITY;
        }
        if (st.tcol >= col0 && st.tcol < col0 + 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j == st.tcol) st.t = v[j];
        }
        float cm = v[0];
#pragma unroll
        for (int j = 1; j < 32; ++j) cm = fmaxf(cm, v[j]);
        const float nm = fmaxf(st.m, cm);
        // nm == -inf only if every logit so far is -inf; keep the exponent arguments finite
        const float nm2 = (nm == -INFINITY) ? 0.f : nm * kLog2e;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) acc += ptx::ex2(fmaf(v[j], kLog2e, -nm2));
        st.s = st.s * ptx::ex2(fmaf(st.m, kLog2e, -nm2)) + acc;
        st.m = nm;
    }
    static __device__ __forceinline__ void end(State& st, const Params& p, const TileCtx& tc) {
        if (st.row < p.rows) {
            float* base = p.partial + static_cast<long long>(tc.n_tile) * 3 * p.row_stride + st.row;
            base[0] = st.m;
            base[p.row_stride] = st.s;
            base[2 * p.row_stride] = st.t;
        }
    }
};

// ---------------------------------------------------------------------------------------------
// Greedy decoding head: per (vocab tile, row) the maximum logit, sum exp(z - max) and the COLUMN of the
// maximum (first one on ties), in the partial layout of EpiStats with the column's bits in the third
// slot. Merged per row this gives argmax_v z[row, v] and its log-probability -log(sum exp(z - max))
// without the logits ever reaching memory. No counterpart in the reference, whose decode step
// materialises the logits through matmul (examples/common.py:127-131, 380-384).
// ---------------------------------------------------------------------------------------------
struct EpiTop1 {
    static constexpr bool kHasFinish = false;
    struct Params {
        int rows;   // valid rows
        int vocab;  // valid columns (local shard width)
        float* partial;
        long long row_stride;
    };
    struct State {
        float m, s;
        int arg;  // local column of the running maximum
        int row;
    };
    static __device__ __forceinline__ void begin(State& st, const Params&, const TileCtx& tc) {
        st.row = tc.m_tile * kBM + tc.row_in_tile;
        st.m = -INFINITY;
        st.s = 0.f;
        st.arg = tc.n_tile * tc.bn;
    }
    static __device__ __forceinline__ void chunk(State& st, const Params& p, const TileCtx& tc,
                                                 int col0, float (&v)[32]) {
        const int gcol0 = tc.n_tile * tc.bn + col0;
        if (gcol0 >= p.vocab) return;
        if (gcol0 + 32 > p.vocab) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (gcol0 + j >= p.vocab) v[j] = -INFINITY;
        }
        float cm = v[0];
        int cj = 0;
#pragma unroll
        for (int j = 1; j < 32; ++j)
            if (v[j] > cm) {  // strict: the first maximum wins
                cm = v[j];
                cj = j;
            }
        if (cm > st.m) st.arg = gcol0 + cj;  // chunks arrive in ascending column order
        const float nm = fmaxf(st.m, cm);
        const float nm2 = (nm == -INFINITY) ? 0.f : nm * kLog2e;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) acc += ptx::ex2(fmaf(v[j], kLog2e, -nm2));
        st.s = st.s * ptx::ex2(fmaf(st.m, kLog2e, -nm2)) + acc;
        st.m = nm;
    }
    static __device__ __forceinline__ void end(State& st, const Params& p, const TileCtx& tc) {
        if (st.row < p.rows) {
            float* base = p.partial + static_cast<long long>(tc.n_tile) * 3 * p.row_stride + st.row;
            base[0] = st.m;
            base[p.row_stride] = st.s;
            base[2 * p.row_stride] = __int_as_float(st.arg);
        }
    }
};

// ---------------------------------------------------------------------------------------------
// Sampling head: per (vocab tile, row) the kTileTop largest SCALED logits y = z * scale (scale = 1 /
// temperature) with their columns, sorted (larger first; on equal values the lower column first), and the
// tile's max / sum exp(y - max). Record layout, kTopRecord floats per (tile, row), component-major like
// EpiStats:   0 max   1 sum-exp   2 .. 2+kTileTop-1 values   2+kTileTop .. columns (int bits, local).
// Slots beyond the tile's valid columns hold -inf / column -1. A per-row merge (merge_topk_kernel) selects
// the k best of all tiles; a tile may hold more than kTileTop of them, which the merge detects (the
// tile's weakest kept entry still outranks the k-th) and repairs by recomputing that tile's logits.
// No counterpart in the reference: its decode step materialises all V logits and calls torch.topk /
// torch.sort on them (examples/common.py:288-301, 380-384).
// ---------------------------------------------------------------------------------------------
constexpr int kTileTop = 8;
constexpr int kTopRecord = 2 + 2 * kTileTop;

struct EpiTopK {
    static constexpr bool kHasFinish = false;
    struct Params {
        int rows;   // valid rows
        int vocab;  // valid columns (local shard width)
        float scale;
        float* partial;
        long long row_stride;
    };
    struct State {
        float m, s;
        float val[kTileTop];
        int col[kTileTop];
        int row;
    };
    static __device__ __forceinline__ void begin(State& st, const Params&, const TileCtx& tc) {
        st.row = tc.m_tile * kBM + tc.row_in_tile;
        st.m = -INFINITY;
        st.s = 0.f;
#pragma unroll
        for (int i = 0; i < kTileTop; ++i) {
            st.val[i] = -INFINITY;
            st.col[i] = -1;
        }
    }
    static __device__ __forceinline__ void chunk(State& st, const Params& p, const TileCtx& tc,
                                                 int col0, float (&v)[32]) {
        const int gcol0 = tc.n_tile * tc.bn + col0;
        if (gcol0 >= p.vocab) return;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (gcol0 + j < p.vocab) ? v[j] * p.scale : -INFINITY;
        float cm = v[0];
#pragma unroll
        for (int j = 1; j < 32; ++j) cm = fmaxf(cm, v[j]);
        if (cm > st.val[kTileTop - 1]) {  // something in this chunk enters the list
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if (v[j] > st.val[kTileTop - 1]) {  // strict: of equal values the earlier column stays
                    st.val[kTileTop - 1] = v[j];
                    st.col[kTileTop - 1] = gcol0 + j;
#pragma unroll
                    for (int i = kTileTop - 2; i >= 0; --i) {
                        if (st.val[i + 1] > st.val[i]) {
                            const float tv = st.val[i];
                            st.val[i] = st.val[i + 1];
                            st.val[i + 1] = tv;
                            const int tcl = st.col[i];
                            st.col[i] = st.col[i + 1];
                            st.col[i + 1] = tcl;
                        }
                    }
                }
            }
        }
        const float nm = fmaxf(st.m, cm);
        const float nm2 = (nm == -INFINITY) ? 0.f : nm * kLog2e;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) acc += ptx::ex2(fmaf(v[j], kLog2e, -nm2));
        st.s = st.s * ptx::ex2(fmaf(st.m, kLog2e, -nm2)) + acc;
        st.m = nm;
    }
    static __device__ __forceinline__ void end(State& st, const Params& p, const TileCtx& tc) {
        if (st.row < p.rows) {
            float* base = p.partial + static_cast<long long>(tc.n_tile) * kTopRecord * p.row_stride + st.row;
            base[0] = st.m;
            base[p.row_stride] = st.s;
#pragma unroll
            for (int i = 0; i < kTileTop; ++i) {
                base[(2 + i) * p.row_stride] = st.val[i];
                base[(2 + kTileTop + i) * p.row_stride] = __int_as_float(st.col[i]);
            }
        }
    }
};

// ---------------------------------------------------------------------------------------------
// Backward step 1: recompute a logits tile and turn it into the logit gradient
//   G[row, col] = (exp(z - lse[row]) - [col == target[row]]) * rowscale[row]
// rounded to the input dtype (the reference rounds G the same way before its two GEMMs,
// tritium/ops/cross_entropy.py:361-367) and written to the band buffer g[row * ldg + col].
// rowscale already holds grad_out / valid_count (or grad_out, or grad_out[row]) and is 0 for
// ignored rows. The GEMM runs on a sub-block (rows row_off.., local columns col_off..).
// ---------------------------------------------------------------------------------------------
template <class T>
struct EpiGrad {
    static constexpr bool kHasFinish = false;
    struct Params {
        const void* tgt;
        int tgt_i64;
        int rows;               // valid rows of this block
        int cols;               // valid columns of this block
        int row_off;            // first global row of the block
        long long col_global0;  // global vocab index of block column 0
        const float* lse;
        const float* rowscale;  // per-row factor, or nullptr: small batches derive it here (fields below)
        T* g;
        long long ldg;
        // rowscale == nullptr: factor = grad_out (one float, or one per row) / valid-row count (mean only), 0 for
        // ignored rows. Every epilogue warp counts the valid targets of all n_total rows itself - a few loads per
        // lane while the tile's main loop runs - which saves small problems a launch.
        const float* grad_out = nullptr;
        int go_per_row = 0, mean = 0, n_total = 0;
        long long ignore_index = -100;
        int wide = 0;  // 16-bit G leaves as whole 128-byte lines (store_block64) where the core provides the area
    };
    struct State {
        float l2, sc;
        int tcol, row;
    };
    static __device__ __forceinline__ void begin(State& st, const Params& p, const TileCtx& tc) {
        st.row = tc.m_tile * kBM + tc.row_in_tile;
        st.tcol = -1;
        st.sc = 0.f;
        st.l2 = 0.f;
        float count = 1.f;
        if (p.rowscale == nullptr && p.mean) {  // all 32 lanes of the warp take part
            int c = 0;
            for (int i = tc.row_in_tile & 31; i < p.n_total; i += 32) c += load_target(p.tgt, p.tgt_i64, i) != p.ignore_index;
            count = static_cast<float>(__reduce_add_sync(0xffffffffu, c));
        }
        if (st.row < p.rows) {
            const int grow = p.row_off + st.row;
            const long long target = load_target(p.tgt, p.tgt_i64, grow);
            if (p.rowscale != nullptr) {
                st.sc = p.rowscale[grow];
            } else if (target != p.ignore_index) {
                const float g = p.go_per_row ? p.grad_out[grow] : p.grad_out[0];
                st.sc = p.mean ? g / count : g;
            }
            st.l2 = p.lse[grow] * kLog2e;
            const long long rel = target - p.col_global0 - static_cast<long long>(tc.n_tile) * tc.bn;
            if (rel >= 0 && rel < tc.bn) st.tcol = static_cast<int>(rel);
        }
    }
    static __device__ __forceinline__ void chunk(State& st, const Params& p, const TileCtx& tc,
                                                 int col0, float (&v)[32]) {
        const int bcol0 = tc.n_tile * tc.bn + col0;  // column inside the block
        bool wide = false;
        if constexpr (sizeof(T) == 2) wide = p.wide != 0 && tc.stage != nullptr;
        if (!wide && (st.row >= p.rows || bcol0 >= p.cols)) return;
        if (st.sc == 0.f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = ptx::ex2(fmaf(v[j], kLog2e, -st.l2)) * st.sc;
            if (st.tcol >= col0 && st.tcol < col0 + 32) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j == st.tcol) v[j] -= st.sc;
            }
        }
        if constexpr (sizeof(T) == 2) {
            if (wide) {  // all 32 lanes, rows or columns past the end included (nothing is stored for those)
                const int lane = tc.row_in_tile & 31, half = (col0 >> 5) & 1;
                const int row_base = st.row - lane, blk0 = bcol0 - half * 32;
                store_block64<T>(tc.stage, lane, half, v, p.g + static_cast<long long>(row_base) * p.ldg + blk0, p.ldg,
                                 p.rows - row_base, p.cols - blk0);
                return;
            }
        }
        store_row32<T>(p.g + static_cast<long long>(st.row) * p.ldg + bcol0, v, p.cols - bcol0);
    }
    static __device__ __forceinline__ void end(State&, const Params&, const TileCtx&) {}
};

// ---------------------------------------------------------------------------------------------
// Backward steps 2 and 3: store a plain GEMM result (dW block or dX block), optionally summed
// over several launches in a fixed order through an fp32 scratch buffer:
//   kStoreDirect  out = acc                      (the contraction was complete in one launch)
//   kStoreFirst   scratch = acc                  (first partial sum)
//   kStoreAccum   scratch += acc
//   kStoreLast    out = scratch + acc            (rounded to the output dtype once, at the end)
//   kStoreSlice   scratch[k_slice] = acc         (split-K inside one launch: each slice of the
//                                                 contraction writes its own slab of slab_floats
//                                                 floats; splitk_reduce_kernel adds the slabs in
//                                                 slice order afterwards)
// The launches of one sum run in stream order, so the summation order - and the result - is the
// same on every run (this is the deterministic split-K). The scratch buffer is private to the
// library, so it is laid out for coalescing, not as a matrix: float4 index
//   ((tile * bn/4 + col/4) * 128 + row_in_tile).
// ---------------------------------------------------------------------------------------------
constexpr int kMaxPeers = 8;

enum StoreMode { kStoreDirect = 0, kStoreFirst = 1, kStoreAccum = 2, kStoreLast = 3, kStoreSlice = 4 };

template <class T>
struct EpiStore {
    static constexpr bool kHasFinish = false;
    struct Params {
        T* out;
        long long ldo;
        int rows, cols;  // valid extent of the output block
        float* scratch;
        int mode;
        long long slab_floats;  // kStoreSlice: distance between the slabs of consecutive k slices
        // Peer scatter (peer_world > 0, T = float only): the finished row does not go to `out` but
        // to the GPU that owns it in a reduce-scatter over row slices. Row g (= row_off + local row)
        // belongs to rank g / rows_per_rank, and lands in that rank's staging buffer
        // [world][rows_per_rank][ldo] in the slot of the sending rank. The stores go over NVLink from
        // inside the GEMM epilogue; nothing waits on another GPU here.
        T* peer[kMaxPeers];
        int peer_world, peer_rank;
        int rows_per_rank;
        int row_off;
        // Optional sum of squares of the FINAL output values as stored (after rounding to T), for the gradient
        // norm: every (tile, warp) writes one partial, sumsq_partial[((sumsq_tile0 + m_tile) * n_tiles + n_tile)
        // * 4 + warp]; a later pass adds the partials in index order. Which CTA computes a tile does not matter,
        // so the total is the same on every run. nullptr = off. Only in the modes that produce final values.
        float* sumsq_partial = nullptr;
        int sumsq_tile0 = 0;
        // 16-bit results leave as whole 128-byte lines (store_block64). The host sets it only when `out` is
        // 16-byte aligned and ldo is a multiple of 8.
        int wide = 0;
    };
    struct State {
        int row;
        T* dst;  // start of this thread's output row
        float sq;
    };
    static __device__ __forceinline__ void begin(State& st, const Params& p, const TileCtx& tc) {
        st.sq = 0.f;
        st.row = tc.m_tile * kBM + tc.row_in_tile;
        if (p.peer_world > 0) {
            const int g = p.row_off + st.row;
            const int owner = g / p.rows_per_rank;
            st.dst = p.peer[owner < p.peer_world ? owner : 0] +
                     (static_cast<long long>(p.peer_rank) * p.rows_per_rank + (g - owner * p.rows_per_rank)) * p.ldo;
        } else {
            st.dst = p.out + static_cast<long long>(st.row) * p.ldo;
        }
    }
    static __device__ __forceinline__ void chunk(State& st, const Params& p, const TileCtx& tc,
                                                 int col0, float (&v)[32]) {
        const int gcol0 = tc.n_tile * tc.bn + col0;
        if (p.mode != kStoreDirect) {
            float4* sp = reinterpret_cast<float4*>(p.scratch) +
                         ((static_cast<long long>(tc.m_tile) * tc.n_tiles + tc.n_tile) * (tc.bn / 4) +
                          col0 / 4) * kBM + tc.row_in_tile;
            if (p.mode == kStoreSlice) sp += static_cast<long long>(tc.k_slice) * (p.slab_floats / 4);
            if (p.mode != kStoreFirst && p.mode != kStoreSlice) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 o = sp[i * kBM];
                    v[4 * i + 0] += o.x;
                    v[4 * i + 1] += o.y;
                    v[4 * i + 2] += o.z;
                    v[4 * i + 3] += o.w;
                }
            }
            if (p.mode != kStoreLast) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    sp[i * kBM] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                return;
            }
        }
        if constexpr (std::is_same<T, float>::value) {
            if (p.peer_world > 0 && tc.stage != nullptr) {
                // Peer rows leave as whole 128-byte lines: the warp re-shapes its 32 x 32 chunk through
                // shared memory so that 8 lanes cover one row (4 columns each) instead of every lane
                // sending 16 bytes of a different row - NVLink carries few large writes far better than
                // many small ones. All 32 lanes take part; rows / columns out of range are skipped.
                const int lane = tc.row_in_tile & 31;
                float* sm = tc.stage;
#pragma unroll
                for (int j = 0; j < 32; ++j) sm[lane * 33 + j] = v[j];
                __syncwarp();
                const int row_base = st.row - lane;
                const int c4 = (lane & 7) * 4;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int r = it * 4 + (lane >> 3);
                    float* dst = reinterpret_cast<float*>(
                        __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(st.dst), r));
                    if (row_base + r < p.rows && gcol0 + c4 + 4 <= p.cols) {
                        const float* src = sm + r * 33 + c4;
                        *reinterpret_cast<float4*>(dst + gcol0 + c4) = make_float4(src[0], src[1], src[2], src[3]);
                    }
                }
                __syncwarp();
                return;
            }
        }
        if constexpr (sizeof(T) == 2) {
            if (p.wide != 0 && tc.stage != nullptr) {  // all 32 lanes take part, whatever their row and column
                const int lane = tc.row_in_tile & 31, half = (col0 >> 5) & 1;
                const int row_base = st.row - lane, blk0 = gcol0 - half * 32;
                store_block64<T>(tc.stage, lane, half, v, p.out + static_cast<long long>(row_base) * p.ldo + blk0, p.ldo,
                                 p.rows - row_base, p.cols - blk0);
                if (p.sumsq_partial != nullptr && st.row < p.rows) {
                    const int valid = p.cols - gcol0;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float r = Cvt<T>::to_f(Cvt<T>::from_f(v[j]));  // the value as stored
                        if (j < valid) st.sq = fmaf(r, r, st.sq);
                    }
                }
                return;
            }
        }
        if (st.row >= p.rows || gcol0 >= p.cols) return;
        store_row32<T>(st.dst + gcol0, v, p.cols - gcol0);
        if (p.sumsq_partial != nullptr) {
            const int valid = p.cols - gcol0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float r = Cvt<T>::to_f(Cvt<T>::from_f(v[j]));  // the value as stored
                if (j < valid) st.sq = fmaf(r, r, st.sq);
            }
        }
    }
    static __device__ __forceinline__ void end(State& st, const Params& p, const TileCtx& tc) {
        if (p.sumsq_partial == nullptr || (p.mode != kStoreDirect && p.mode != kStoreLast)) return;
        float sq = st.sq;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
        if ((tc.row_in_tile & 31) == 0 && tc.m_tile * kBM < p.rows)
            p.sumsq_partial[(static_cast<long long>(p.sumsq_tile0 + tc.m_tile) * tc.n_tiles + tc.n_tile) * 4 +
                            (tc.row_in_tile >> 5)] = sq;
    }
};

}  // namespace lce
