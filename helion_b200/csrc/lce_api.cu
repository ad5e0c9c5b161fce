// extern "C" entry points of libhelion_lce.so (declared in include/helion_lce.h): argument checks,
// tensor-map construction, the block plan of the backward pass, and the kernel launches.
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "../../include/helion_lce.h"
#include "gemm_simt.cuh"
#include "gemm_tc.cuh"
#include "ce_kernels.cuh"
#include "norm_kernels.cuh"
#include "optim_kernels.cuh"
#include "row_kernels.cuh"
#include "topk_kernels.cuh"

namespace lce {

__device__ int g_device_status = 0;
// Completion counters of launches whose last CTA runs a fused tail (gemm_tc_kernel, done_counter). A launch takes
// the next slot in turn; the counter returns to zero with the launch's last CTA, so a slot is ready for re-use
// long before the turn comes round to it again (kDoneSlots launches later).
constexpr int kDoneSlots = 4096;
__device__ unsigned g_done_counters[kDoneSlots];

namespace {

constexpr int kBN = 256;
constexpr int kStages1 = 4;  // 48 KB stages, one CTA per tile
constexpr int kStages2 = 6;  // 32 KB stages, CTA pair per tile
constexpr size_t kDefaultBlockBytes = 256ull << 20;
constexpr int kMaxDevices = 64;

struct DeviceInfo {
    bool ready = false;
    int index = 0;
    int sm_count = 0;
    int cc_major = 0;
    int* status_ptr = nullptr;
    unsigned* done_counters = nullptr;  // kDoneSlots of them, zero when idle
    mutable std::atomic<unsigned> next_done_slot{0};
};

DeviceInfo g_dev[kMaxDevices];
std::mutex g_mutex;
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::atomic<unsigned long long> g_launches{0};  // kernels this library has launched (all devices)
#define LCE_COUNT_LAUNCH() g_launches.fetch_add(1, std::memory_order_relaxed)

// The CUDA error behind the last LCE_ERR_CUDA of this thread (lce_last_cuda_error reports its name).
thread_local cudaError_t t_last_cuda_error = cudaSuccess;
inline bool cuda_failed(cudaError_t e) {
    if (e == cudaSuccess) return false;
    t_last_cuda_error = e;
    return true;
}

int device_info(DeviceInfo** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return LCE_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return LCE_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo& d = g_dev[dev];
    if (!d.ready) {
        d.index = dev;
        if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return LCE_ERR_CUDA;
        if (cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
            return LCE_ERR_CUDA;
        if (d.cc_major == 10) {
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return LCE_ERR_CUDA;
            d.status_ptr = static_cast<int*>(p);
            if (cudaGetSymbolAddress(&p, g_done_counters) != cudaSuccess) return LCE_ERR_CUDA;
            d.done_counters = static_cast<unsigned*>(p);
        }
        d.ready = true;
    }
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || fn == nullptr)
            return LCE_ERR_CUDA;
        g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    *out = &d;
    return d.cc_major == 10 ? LCE_OK : LCE_ERR_ARCH;
}

inline long long cdiv(long long a, long long b) { return (a + b - 1) / b; }
inline size_t align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }
inline size_t elem_size(int dtype) { return dtype == LCE_DTYPE_F32 ? 4 : 2; }

// 2-D tensor map over a row-major 16-bit matrix: `inner` contiguous elements per row, `outer`
// rows, `pitch_bytes` between rows; 128-byte swizzle; out-of-range elements read as zero.
// Encoding is host-only work (no driver state is touched), but it costs about a microsecond per map and
// a training step issues the same handful of maps over and over, so finished maps are kept in a small
// per-thread, direct-mapped cache keyed by everything the encoding depends on.
struct TmapKey {
    const void* base;
    long long inner, outer, pitch_bytes;
    unsigned box_inner, box_outer;
    int dtype;
    bool operator==(const TmapKey& o) const {
        return base == o.base && inner == o.inner && outer == o.outer && pitch_bytes == o.pitch_bytes &&
               box_inner == o.box_inner && box_outer == o.box_outer && dtype == o.dtype;
    }
};
struct TmapSlot {
    TmapKey key;
    bool valid = false;
    CUtensorMap map;
};
constexpr int kTmapCacheSlots = 64;

int make_tmap(CUtensorMap* tm, const void* base, int dtype, long long inner, long long outer,
              long long pitch_bytes, unsigned box_inner, unsigned box_outer) {
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (pitch_bytes & 15) != 0) return LCE_ERR_ALIGN;
    static thread_local TmapSlot cache[kTmapCacheSlots];
    const TmapKey key{base, inner, outer, pitch_bytes, box_inner, box_outer, dtype};
    unsigned long long h = reinterpret_cast<uintptr_t>(base) >> 4;
    h = h * 0x9E3779B97F4A7C15ull ^ static_cast<unsigned long long>(inner) * 0xC2B2AE3D27D4EB4Full ^
        static_cast<unsigned long long>(outer) * 0x165667B19E3779F9ull ^ (static_cast<unsigned long long>(box_outer) << 7) ^
        static_cast<unsigned long long>(pitch_bytes);
    TmapSlot& slot = cache[(h ^ (h >> 29)) % kTmapCacheSlots];
    if (slot.valid && slot.key == key) {
        *tm = slot.map;
        return LCE_OK;
    }
    // The encoder is a DRIVER entry point and wants a context current on the calling thread. A thread that has
    // made no runtime call yet (an autograd worker whose first CUDA call is this one) has none bound, and the
    // encoder then fails with CUDA_ERROR_INVALID_CONTEXT. cudaSetDevice on the thread's current device binds
    // the primary context (and, unlike cudaFree(0), is no stream operation, so it is legal under stream capture).
    {
        static thread_local int bound_device = -1;
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && dev != bound_device && cudaSetDevice(dev) == cudaSuccess) bound_device = dev;
    }
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_bytes)};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt =
        dtype == LCE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult r = g_encode(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        t_last_cuda_error = static_cast<cudaError_t>(r);  // driver and runtime share the numbering of the common codes
        if (getenv("HELION_B200_DEBUG"))
            fprintf(stderr, "helion_b200: cuTensorMapEncodeTiled failed (%d): base %p inner %lld outer %lld pitch %lld box %u x %u\n",
                    static_cast<int>(r), base, inner, outer, pitch_bytes, box_inner, box_outer);
        return LCE_ERR_CUDA;
    }
    slot.key = key;
    slot.map = *tm;
    slot.valid = true;
    return LCE_OK;
}

// One operand of a GEMM as the host sees it: a row-major matrix [rows, cols] with a pitch.
// As a K-major operand its rows are the m (n) index; as an MN-major operand its rows are k.
struct Mat {
    const void* ptr;
    long long rows, cols, pitch_elems;
};

// Tuning knobs of the tcgen05 launches (environment at load time, lce_set_tuning at run time):
//   band_mb     size of the operand band the tile order keeps resident in L2 (HELION_B200_BAND_MB)
//   hint_mode   L2 eviction hints: 0 none, 1 resident operand evict_last + streaming evict_first,
//               2 evict_last only (HELION_B200_L2_HINTS)
//   dyn_waves   launches of at least this many waves of tiles deal their tiles dynamically, when the caller's
//               workspace has room for the counter; 0 = never (HELION_B200_DYN_WAVES). 32: the long forward
//               launches, where the static deal drifts apart; the backward's launches are capped at about 28
//               waves by the block size and measured 1 % faster on the static deal
struct Tuning {
    std::atomic<int> band_mb, hint_mode, dyn_waves;
    Tuning() {
        const char* e = getenv("HELION_B200_BAND_MB");
        band_mb = (e && atoi(e) > 0) ? atoi(e) : 32;
        e = getenv("HELION_B200_L2_HINTS");
        hint_mode = e ? atoi(e) : 2;
        e = getenv("HELION_B200_DYN_WAVES");
        dyn_waves = e ? atoi(e) : 32;
    }
};
Tuning g_tuning;

// Programmatic dependent launch (HELION_B200_PDL=0 switches it off): kernels that call ptx::grid_dep_wait()
// before they read anything their predecessor in the stream wrote may be launched while that predecessor is
// still running; their launch latency and set-up then hide under its tail.
inline bool pdl_enabled() {
    static const bool kEnabled = [] { const char* e = getenv("HELION_B200_PDL"); return e ? atoi(e) != 0 : true; }();
    return kEnabled;
}

// Launches such a kernel (no dynamic shared memory). Only for kernels that contain the wait.
template <class... KArgs, class... Args>
cudaError_t launch_dependent(void (*kern)(KArgs...), int grid, int block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <int CG, bool A_MN, bool B_MN, bool IS_BF16, class Epi>
int launch_tc_cg(const DeviceInfo& d, const Mat& a, const Mat& b, long long M, long long Nn, long long K,
                 int m_fastest, int k_splits, const typename Epi::Params& ep, cudaStream_t stream, int* sched,
                 unsigned* done) {
    // Band the tile order so that the panels which co-running CTAs do NOT share stay resident in L2:
    // about 32 MB of them (the two L2 partitions of 63 MB each also hold the streaming operand).
    const long long kBandBytes = static_cast<long long>(g_tuning.band_mb.load(std::memory_order_relaxed)) << 20;
    const int kHintMode = g_tuning.hint_mode.load(std::memory_order_relaxed);
    constexpr int kStages = CG == 2 ? kStages2 : kStages1;
    const int dtype = IS_BF16 ? LCE_DTYPE_BF16 : LCE_DTYPE_F16;
    CUtensorMap tma, tmb;
    int rc;
    if (A_MN) rc = make_tmap(&tma, a.ptr, dtype, M, K, a.pitch_elems * 2, 64, kBK);
    else rc = make_tmap(&tma, a.ptr, dtype, K, M, a.pitch_elems * 2, kBK, kBM);
    if (rc) return rc;
    // each CTA of a pair stages half of the B tile
    if (B_MN) rc = make_tmap(&tmb, b.ptr, dtype, Nn, K, b.pitch_elems * 2, 64, kBK);
    else rc = make_tmap(&tmb, b.ptr, dtype, K, Nn, b.pitch_elems * 2, kBK, kBN / CG);
    if (rc) return rc;
    const long long m_tiles = cdiv(M, kBM), n_tiles = cdiv(Nn, kBN), k_blocks = cdiv(K, kBK);
    const long long units = cdiv(m_tiles, CG) * n_tiles;
    if (m_tiles * n_tiles > 0x3fffffffll || k_blocks > 0x7fffffffll) return LCE_ERR_TOO_LARGE;
    if (units == 0 || k_blocks == 0) return LCE_OK;
    // every k slice must hold at least one block
    if (k_splits < 1 || (k_splits - 1) * cdiv(k_blocks, k_splits) >= k_blocks) return LCE_ERR_ARG;
    auto kern = gemm_tc_kernel<kBN, kStages, CG, A_MN, B_MN, IS_BF16, Epi>;
    constexpr int smem = GemmSmem<kBN, kStages, CG>::kTotalBytes;
    // per kernel instantiation and device; setting the attribute twice from two threads is harmless
    static std::atomic<bool> smem_opted_in[kMaxDevices];
    if (!smem_opted_in[d.index].load(std::memory_order_acquire)) {
        if (cuda_failed(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
            return LCE_ERR_CUDA;
        smem_opted_in[d.index].store(true, std::memory_order_release);
    }
    const long long slots = d.sm_count / CG;  // one CTA per SM; a pair occupies the two SMs of a TPC
    const long long work = units * k_splits;
    const int grid = static_cast<int>(work < slots ? work : slots) * CG;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    // The kernel waits for its predecessor in the stream itself (ptx::grid_dep_wait after its set-up), so it may
    // be started under the predecessor's tail; pairs additionally launch as clusters of two.
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (CG > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = CG;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    // the banded operand is re-read by every tile of the band: keep it; the other one streams
    const int stream_hint = kHintMode == 1 ? ptx::kL2EvictFirst : ptx::kL2Normal;
    const int l2_hints = kHintMode == 0 ? 0 : (m_fastest ? (ptx::kL2EvictLast | (stream_hint << 2))
                                                          : (stream_hint | (ptx::kL2EvictLast << 2)));
    int raster;
    if (m_fastest) {  // bands of row units: rows fastest inside
        long long wb = kBandBytes / (static_cast<long long>(CG) * kBM * K * 2);
        const long long m_units = cdiv(m_tiles, CG);
        raster = static_cast<int>(wb < 1 ? 1 : (wb > m_units ? m_units : wb));
    } else {  // bands of tile columns: columns fastest inside
        long long wb = kBandBytes / (static_cast<long long>(kBN) * K * 2);
        raster = -static_cast<int>(wb < 1 ? 1 : (wb > n_tiles ? n_tiles : wb));
    }
    // Long launches deal their tiles from a counter in the caller's workspace, zeroed in stream order here.
    const int dyn_waves = g_tuning.dyn_waves.load(std::memory_order_relaxed);
    int* counter = (sched != nullptr && dyn_waves > 0 && work >= dyn_waves * slots) ? sched : nullptr;
    if (counter != nullptr && cuda_failed(cudaMemsetAsync(counter, 0, sizeof(int), stream))) return LCE_ERR_CUDA;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, tma, tmb, static_cast<int>(m_tiles),
                                               static_cast<int>(n_tiles), static_cast<int>(k_blocks), k_splits,
                                               raster, l2_hints, ep, d.status_ptr, counter, done, NoSecondGemm{});
    LCE_COUNT_LAUNCH();
    return cuda_failed(err) ? LCE_ERR_CUDA : LCE_OK;
}

// Two independent products with the same epilogue kind in ONE launch of single-CTA tiles: the first with a
// K-major A operand, the second with an MN-major one, both with MN-major B (the backward's dX = G W and
// dW = G^T X). Work items of the second follow those of the first in the round-robin deal.
struct GemmProblem {
    Mat a, b;
    long long M, Nn, K;
    int k_splits;
};
template <bool IS_BF16, class Epi>
int launch_tc_two(const DeviceInfo& d, const GemmProblem& p1, const typename Epi::Params& ep1, const GemmProblem& p2,
                  const typename Epi::Params& ep2, cudaStream_t stream) {
    constexpr int dtype = IS_BF16 ? LCE_DTYPE_BF16 : LCE_DTYPE_F16;
    using Second = SecondGemm<Epi, true>;
    CUtensorMap tma1, tmb1;
    Second sec;
    int rc;
    if ((rc = make_tmap(&tma1, p1.a.ptr, dtype, p1.K, p1.M, p1.a.pitch_elems * 2, kBK, kBM))) return rc;      // K-major A
    if ((rc = make_tmap(&tmb1, p1.b.ptr, dtype, p1.Nn, p1.K, p1.b.pitch_elems * 2, 64, kBK))) return rc;       // MN-major B
    if ((rc = make_tmap(&sec.tmA, p2.a.ptr, dtype, p2.M, p2.K, p2.a.pitch_elems * 2, 64, kBK))) return rc;    // MN-major A
    if ((rc = make_tmap(&sec.tmB, p2.b.ptr, dtype, p2.Nn, p2.K, p2.b.pitch_elems * 2, 64, kBK))) return rc;   // MN-major B
    const long long mt1 = cdiv(p1.M, kBM), nt1 = cdiv(p1.Nn, kBN), kb1 = cdiv(p1.K, kBK);
    const long long mt2 = cdiv(p2.M, kBM), nt2 = cdiv(p2.Nn, kBN), kb2 = cdiv(p2.K, kBK);
    if (mt1 * nt1 * p1.k_splits + mt2 * nt2 * p2.k_splits > 0x3fffffffll) return LCE_ERR_TOO_LARGE;
    if (mt1 * nt1 == 0 || mt2 * nt2 == 0 || kb1 == 0 || kb2 == 0) return LCE_ERR_ARG;
    if (p1.k_splits < 1 || (p1.k_splits - 1) * cdiv(kb1, p1.k_splits) >= kb1) return LCE_ERR_ARG;
    if (p2.k_splits < 1 || (p2.k_splits - 1) * cdiv(kb2, p2.k_splits) >= kb2) return LCE_ERR_ARG;
    sec.m_tiles = static_cast<int>(mt2);
    sec.n_tiles = static_cast<int>(nt2);
    sec.k_blocks = static_cast<int>(kb2);
    sec.k_splits = p2.k_splits;
    sec.raster = -static_cast<int>(nt2);  // columns fastest: small problems, everything stays in L2
    sec.ep = ep2;
    auto kern = gemm_tc_kernel<kBN, kStages1, 1, false, true, IS_BF16, Epi, Second>;
    constexpr int smem = GemmSmem<kBN, kStages1, 1>::kTotalBytes;
    static std::atomic<bool> smem_opted_in[kMaxDevices];
    if (!smem_opted_in[d.index].load(std::memory_order_acquire)) {
        if (cuda_failed(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem))) return LCE_ERR_CUDA;
        smem_opted_in[d.index].store(true, std::memory_order_release);
    }
    const long long work = mt1 * nt1 * p1.k_splits + mt2 * nt2 * p2.k_splits;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(work < d.sm_count ? work : d.sm_count));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, tma1, tmb1, static_cast<int>(mt1), static_cast<int>(nt1),
                                               static_cast<int>(kb1), p1.k_splits, -static_cast<int>(nt1), 0, ep1,
                                               d.status_ptr, static_cast<int*>(nullptr),
                                               static_cast<unsigned*>(nullptr), sec);
    LCE_COUNT_LAUNCH();
    return cuda_failed(err) ? LCE_ERR_CUDA : LCE_OK;
}

// CTA pairs cover two 128-row tiles at a time; with an odd, small number of row tiles the second
// half of the last pair would idle, so such problems run on single CTAs.
bool use_pair(long long M, int cg) {
    const long long m_tiles = cdiv(M, kBM);
    return cg == 2 && (m_tiles % 2 == 0 || m_tiles >= 16);
}

// Which tcgen05 variant a call asks for: CTA pairs (cta_group::2) unless LCE_FLAG_ONE_CTA is set.
inline int cta_group_of(unsigned flags) { return (flags & LCE_FLAG_ONE_CTA) ? 1 : 2; }

// Kernel family of one call, decided once from the arguments and passed down (no per-thread state).
struct Path {
    bool use_tc;  // tcgen05 GEMM core (else the CUDA-core one)
    int cg;       // cta group asked for: 2 = CTA pairs, 1 = single CTAs
    int* sched = nullptr;  // 4 bytes of the call's workspace for the dynamic tile deal, or nullptr
};

template <bool A_MN, bool B_MN, bool IS_BF16, class Epi>
int launch_tc(const DeviceInfo& d, int cg, const Mat& a, const Mat& b, long long M, long long Nn, long long K,
              int m_fastest, const typename Epi::Params& ep, cudaStream_t stream, int k_splits = 1,
              int* sched = nullptr, unsigned* done = nullptr) {
    if (use_pair(M, cg))
        return launch_tc_cg<2, A_MN, B_MN, IS_BF16, Epi>(d, a, b, M, Nn, K, m_fastest, k_splits, ep, stream, sched, done);
    return launch_tc_cg<1, A_MN, B_MN, IS_BF16, Epi>(d, a, b, M, Nn, K, m_fastest, k_splits, ep, stream, sched, done);
}

// The same for the CUDA-core GEMM (128 x 128 tiles, two CTAs per SM worth of work items).
int choose_k_splits_simt(long long M, long long Nn, long long K) {
    const long long units = cdiv(M, kBM) * cdiv(Nn, kSimtBN);
    if (units == 0 || units * 2 > 296) return 1;
    long long s = 296 / units;
    if (s > 32) s = 32;
    while (s > 1 && (K / s < 64 || (s - 1) * (cdiv(cdiv(K, s), kSimtBK) * kSimtBK) >= K)) --s;
    return static_cast<int>(s);
}

// How many slices to cut the contraction of an M x Nn x K GEMM into so that a problem with few output
// tiles still fills the GPU (the deterministic split-K: slices are added in slice order afterwards).
// Uses a fixed SM count so that workspace sizes do not depend on the device.
int choose_k_splits(long long M, long long Nn, long long K, int cg) {
    const long long slots = use_pair(M, cg) ? 74 : 148;
    const long long units = cdiv(cdiv(M, kBM), use_pair(M, cg) ? 2 : 1) * cdiv(Nn, kBN);
    const long long k_blocks = cdiv(K, kBK);
    if (units == 0 || units * 2 > slots) return 1;
    long long s = slots / units;
    if (s > 16) s = 16;
    while (s > 1 && (k_blocks / s < 16 || (s - 1) * cdiv(k_blocks, s) >= k_blocks)) --s;
    return static_cast<int>(s);
}

template <class T, class Epi>
int launch_simt(const DeviceInfo& d, const Mat& a, bool a_mn, const Mat& b, bool b_mn, long long M,
                long long Nn, long long K, const typename Epi::Params& ep, cudaStream_t stream, int k_splits = 1) {
    SimtOperand<T> A, B;
    A.ptr = static_cast<const T*>(a.ptr);
    A.stride_mn = a_mn ? 1 : a.pitch_elems;
    A.stride_k = a_mn ? a.pitch_elems : 1;
    A.extent_mn = static_cast<int>(M);
    B.ptr = static_cast<const T*>(b.ptr);
    B.stride_mn = b_mn ? 1 : b.pitch_elems;
    B.stride_k = b_mn ? b.pitch_elems : 1;
    B.extent_mn = static_cast<int>(Nn);
    const long long m_tiles = cdiv(M, kBM), n_tiles = cdiv(Nn, kSimtBN);
    if (m_tiles * n_tiles > 0x7fffffffll) return LCE_ERR_TOO_LARGE;
    if (m_tiles * n_tiles == 0 || K == 0) return LCE_OK;
    const long long cap = static_cast<long long>(d.sm_count) * 4;
    const long long work = m_tiles * n_tiles * k_splits;
    const int grid = static_cast<int>(work < cap ? work : cap);
    const int k = static_cast<int>(K), mt = static_cast<int>(m_tiles), nt = static_cast<int>(n_tiles);
    bool launched = false;
    if constexpr (std::is_same<T, float>::value) {
        // fp32 operands that allow 16-byte loads along their contiguous direction take the vector loaders
        const auto mode = [&](const SimtOperand<float>& op, long long extent) {
            if ((reinterpret_cast<uintptr_t>(op.ptr) & 15u) != 0) return static_cast<int>(kSimtGeneric);
            if (op.stride_k == 1 && op.stride_mn % 4 == 0 && K % 4 == 0) return static_cast<int>(kSimtVecK);
            if (op.stride_mn == 1 && op.stride_k % 4 == 0 && extent % 4 == 0) return static_cast<int>(kSimtVecMN);
            return static_cast<int>(kSimtGeneric);
        };
        const int am = mode(A, M), bm = mode(B, Nn);
#define LCE_SIMT_GO(AM, BM) \
    gemm_simt_kernel<float, Epi, AM, BM><<<grid, kSimtThreads, 0, stream>>>(A, B, k, mt, nt, k_splits, ep), launched = true
        if (am == kSimtVecK && bm == kSimtVecK) LCE_SIMT_GO(kSimtVecK, kSimtVecK);
        else if (am == kSimtVecK && bm == kSimtVecMN) LCE_SIMT_GO(kSimtVecK, kSimtVecMN);
        else if (am == kSimtVecMN && bm == kSimtVecK) LCE_SIMT_GO(kSimtVecMN, kSimtVecK);
        else if (am == kSimtVecMN && bm == kSimtVecMN) LCE_SIMT_GO(kSimtVecMN, kSimtVecMN);
#undef LCE_SIMT_GO
    }
    if (!launched) gemm_simt_kernel<T, Epi><<<grid, kSimtThreads, 0, stream>>>(A, B, k, mt, nt, k_splits, ep);
    LCE_COUNT_LAUNCH();
    return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The tcgen05 path needs 16-bit inputs, 16-byte aligned bases and row pitches (H % 8 == 0).
int choose_path(int dtype, long long H, const void* x, const void* w, unsigned flags, bool* use_tc) {
    const bool can_tc = dtype != LCE_DTYPE_F32 && (H % 8) == 0 && aligned16(x) && aligned16(w);
    if (flags & LCE_FLAG_FORCE_TC) {
        if (flags & LCE_FLAG_FORCE_SIMT) return LCE_ERR_ARG;
        if (dtype == LCE_DTYPE_F32) return LCE_ERR_ARG;
        if (!can_tc) return LCE_ERR_ALIGN;
        *use_tc = true;
        return LCE_OK;
    }
    *use_tc = can_tc && !(flags & LCE_FLAG_FORCE_SIMT);
    return LCE_OK;
}

int check_dims(long long N, long long H, long long V, int dtype) {
    if (N < 0 || H <= 0 || V <= 0) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_F32) return LCE_ERR_ARG;
    if (N > 0x7fffff00ll || H > 0x7fffff00ll || V > 0x7fffff00ll) return LCE_ERR_TOO_LARGE;
    return LCE_OK;
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
struct FwdLayout {
    long long n_tiles, row_stride;
    size_t bytes;
};
FwdLayout fwd_layout(long long N, long long V, bool use_tc) {
    FwdLayout l;
    l.n_tiles = cdiv(V, use_tc ? kBN : kSimtBN);
    l.row_stride = static_cast<long long>(align_up(static_cast<size_t>(N), 64));
    l.bytes = static_cast<size_t>(l.n_tiles) * 3 * l.row_stride * sizeof(float);
    return l;
}

// HELION_B200_FUSED_TAIL=0 (tuning knob) keeps the forward tail of very small problems in its own launch.
inline bool fused_tail_enabled() {
    static const bool kEnabled = [] { const char* e = getenv("HELION_B200_FUSED_TAIL"); return e ? atoi(e) != 0 : true; }();
    return kEnabled;
}

// What follows the logits GEMM: either the merged statistics of this shard (for a cross-shard merge)
// or, when the shard is the whole vocabulary, logsumexp and per-row loss straight away.
struct FwdOutputs {
    float* stats = nullptr;      // [3][N]
    float* lse = nullptr;        // [N]       (fused finalize)
    float* loss_rows = nullptr;  // [N]       (fused finalize)
    long long ignore_index = -100;
    // small batches: merge + finalize + loss reduction in one launch (then loss_rows is not used)
    bool one_launch_tail = false;
    int reduction = LCE_REDUCTION_MEAN;
    float* loss = nullptr;         // () or [N]
    float* valid_count = nullptr;  // optional
};

template <class T>
int forward_stats_impl(const DeviceInfo& d, const Path& path, const void* x, const void* w, const void* tgt,
                       int tgt_i64, long long N, long long H, long long V, long long vocab_start,
                       const FwdOutputs& out, void* ws, cudaStream_t stream) {
    const bool use_tc = path.use_tc;
    const int cg = path.cg;
    const FwdLayout l = fwd_layout(N, V, use_tc);
    EpiStats::Params ep;
    ep.tgt = tgt;
    ep.tgt_i64 = tgt_i64;
    ep.rows = static_cast<int>(N);
    ep.vocab = static_cast<int>(V);
    ep.vocab_start = vocab_start;
    ep.partial = static_cast<float*>(ws);
    ep.row_stride = l.row_stride;
    const Mat a{x, N, H, H}, b{w, V, H, H};
    int rc;
    // Very small problems: the GEMM launch's last CTA does the tail itself (EpiStats::finish) - one launch in all.
    // Its 192 threads fold a row's tiles one after the other, so this is only for few rows x few tiles.
    unsigned* done = nullptr;
    // Not while the stream is being captured: a graph would carry its counter into every replay, where it could
    // meet a later launch that was dealt the same one.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (out.one_launch_tail && use_tc && fused_tail_enabled() && N * l.n_tiles <= 4096 &&
        cudaStreamIsCapturing(stream, &capturing) == cudaSuccess && capturing == cudaStreamCaptureStatusNone) {
        ep.fin_lse = out.lse;
        ep.fin_loss = out.loss;
        ep.fin_valid_count = out.valid_count;
        ep.fin_reduction = out.reduction;
        ep.fin_ignore_index = out.ignore_index;
        ep.fin_n_tiles = static_cast<int>(l.n_tiles);
        done = d.done_counters + d.next_done_slot.fetch_add(1, std::memory_order_relaxed) % kDoneSlots;
    }
    if (use_tc) {
        if constexpr (sizeof(T) == 2) {
            constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
            rc = launch_tc<false, false, kBf16, EpiStats>(d, cg, a, b, N, V, H, /*rows first: bands of X stay in L2, W streams*/ 1, ep, stream, 1, path.sched, done);
        } else {
            rc = LCE_ERR_ARG;
        }
    } else {
        rc = launch_simt<T, EpiStats>(d, a, false, b, false, N, V, H, ep, stream);
    }
    if (rc) return rc;
    if (done != nullptr) return LCE_OK;
    const int blocks = static_cast<int>(cdiv(N, kMergeRows)), threads = kMergeRows * kMergeLanes;
    cudaError_t err;
    if (out.one_launch_tail)
        err = launch_dependent(merge_finalize_small_kernel, 1, 1024, stream,
                               static_cast<const float*>(ws), static_cast<int>(l.n_tiles), l.row_stride, static_cast<int>(N),
                               tgt, tgt_i64, out.ignore_index, out.reduction, out.lse, out.loss, out.valid_count);
    else if (out.stats != nullptr)
        err = launch_dependent(merge_partials_kernel<false>, blocks, threads, stream,
                               static_cast<const float*>(ws), static_cast<int>(l.n_tiles), l.row_stride, static_cast<int>(N),
                               out.stats, static_cast<const void*>(nullptr), 0, 0ll, static_cast<float*>(nullptr),
                               static_cast<float*>(nullptr));
    else
        err = launch_dependent(merge_partials_kernel<true>, blocks, threads, stream,
                               static_cast<const float*>(ws), static_cast<int>(l.n_tiles), l.row_stride, static_cast<int>(N),
                               static_cast<float*>(nullptr), tgt, tgt_i64, out.ignore_index, out.lse, out.loss_rows);
    LCE_COUNT_LAUNCH();
    return cuda_failed(err) ? LCE_ERR_CUDA : LCE_OK;
}

// Greedy head: the forward GEMM with the argmax epilogue, then the per-row merge.
template <class T>
int greedy_head_impl(const DeviceInfo& d, const Path& path, const void* x, const void* w, long long N, long long H,
                     long long V, long long vocab_start, long long* token, float* logprob, float* lse, void* ws,
                     cudaStream_t stream) {
    const bool use_tc = path.use_tc;
    const int cg = path.cg;
    const FwdLayout l = fwd_layout(N, V, use_tc);
    EpiTop1::Params ep;
    ep.rows = static_cast<int>(N);
    ep.vocab = static_cast<int>(V);
    ep.partial = static_cast<float*>(ws);
    ep.row_stride = l.row_stride;
    const Mat a{x, N, H, H}, b{w, V, H, H};
    int rc;
    if (use_tc) {
        if constexpr (sizeof(T) == 2) {
            constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
            rc = launch_tc<false, false, kBf16, EpiTop1>(d, cg, a, b, N, V, H, 1, ep, stream, 1, path.sched);
        } else {
            rc = LCE_ERR_ARG;
        }
    } else {
        rc = launch_simt<T, EpiTop1>(d, a, false, b, false, N, V, H, ep, stream);
    }
    if (rc) return rc;
    const cudaError_t err = launch_dependent(
        merge_top1_kernel, static_cast<int>(cdiv(N, kMergeRows)), kMergeRows * kMergeLanes, stream,
        static_cast<const float*>(ws), static_cast<int>(l.n_tiles), l.row_stride, static_cast<int>(N), vocab_start,
        token, logprob, lse);
    LCE_COUNT_LAUNCH();
    return cuda_failed(err) ? LCE_ERR_CUDA : LCE_OK;
}

// Sampling head: the forward GEMM with the top-candidates epilogue, then the per-row selection.
size_t topk_partial_bytes(long long N, long long V, bool use_tc) {
    const FwdLayout l = fwd_layout(N, V, use_tc);
    return static_cast<size_t>(l.n_tiles) * kTopRecord * l.row_stride * sizeof(float);
}

template <class T>
int topk_head_impl(const DeviceInfo& d, const Path& path, const void* x, const void* w, long long N, long long H,
                   long long V, long long vocab_start, int K, float scale, float* top_val, long long* top_idx,
                   float* lse, void* ws, cudaStream_t stream) {
    const bool use_tc = path.use_tc;
    const int cg = path.cg;
    const FwdLayout l = fwd_layout(N, V, use_tc);
    EpiTopK::Params ep;
    ep.rows = static_cast<int>(N);
    ep.vocab = static_cast<int>(V);
    ep.scale = scale;
    ep.partial = static_cast<float*>(ws);
    ep.row_stride = l.row_stride;
    const Mat a{x, N, H, H}, b{w, V, H, H};
    int rc;
    if (use_tc) {
        if constexpr (sizeof(T) == 2) {
            constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
            rc = launch_tc<false, false, kBf16, EpiTopK>(d, cg, a, b, N, V, H, 1, ep, stream, 1, path.sched);
        } else {
            rc = LCE_ERR_ARG;
        }
    } else {
        rc = launch_simt<T, EpiTopK>(d, a, false, b, false, N, V, H, ep, stream);
    }
    if (rc) return rc;
    const cudaError_t err = launch_dependent(
        merge_topk_kernel<T>, static_cast<int>(N), kTopkThreads, stream,
        static_cast<const float*>(ws), static_cast<int>(l.n_tiles), use_tc ? kBN : kSimtBN, l.row_stride,
        static_cast<int>(N), static_cast<const T*>(x), static_cast<const T*>(w), static_cast<int>(H),
        static_cast<int>(V), scale, vocab_start, K, top_val, top_idx, lse);
    LCE_COUNT_LAUNCH();
    return cuda_failed(err) ? LCE_ERR_CUDA : LCE_OK;
}

// ---------------------------------------------------------------------------------------------
// backward block plan
// ---------------------------------------------------------------------------------------------
// G = dLoss/dLogits is produced one block [nr rows x nc vocab columns] at a time and consumed at
// once by the dW and dX GEMMs. A block spanning all rows (vocab bands) completes dW[band] in one
// launch and sums dX over bands; a block spanning the whole vocabulary (row chunks) completes
// dX[chunk] and sums dW over chunks; in general the blocks form a 2-D grid and both are summed.
// The plan takes the block shape under the byte cap that moves the fewest fp32 partial sums.
struct BwdPlan {
    long long nr, nc;          // block shape (last blocks may be smaller)
    long long n_rblk, n_cblk;  // number of row chunks / vocab bands
    long long ldg;             // pitch of the G block in elements
    long long bn;              // tile width of the dX / dW GEMMs (for the scratch layout)
    size_t off_count, off_rowscale, off_g, off_dx_scratch, off_dw_scratch, off_sumsq, total;
    long long sumsq_floats;      // partial sums of squares of dW: one per (128-row tile, tile column, warp)
    long long dw_band_scratch_floats;
    int dx_splits;               // k slices of the dX GEMM when one band covers the vocabulary
    long long dx_slab_floats;    // fp32 scratch of one dX row chunk (one slice)
    int dw_splits;               // k slices of the dW GEMM when one chunk covers all rows (short vocabulary)
};

BwdPlan plan_backward(long long N, long long H, long long V, int dtype, bool use_tc, unsigned flags,
                      size_t block_bytes) {
    BwdPlan p{};
    const size_t e = elem_size(dtype);
    const size_t cap = block_bytes ? block_bytes : kDefaultBlockBytes;
    const long long col_q = 256, row_q = 128;
    const bool need_dx = !(flags & LCE_FLAG_NO_DX), need_dw = !(flags & LCE_FLAG_NO_DW);
    if (static_cast<size_t>(N) * V * e <= cap || N == 0) {
        p.nr = N > 0 ? N : 1;
        p.nc = V;
    } else {
        // Candidates: all rows, or 128 * 2^k rows; the band is as wide as the cap then allows
        // (multiples of 256 columns, at least 256). Cost = bytes of fp32 partial sums re-read and
        // re-written: dX once per extra vocab band, dW once per extra row chunk.
        double best = 1e300;
        for (long long nr = N;;) {
            long long nc = static_cast<long long>(cap / (static_cast<size_t>(nr) * e)) / col_q * col_q;
            if (nc < col_q) nc = col_q;
            if (nc > V) nc = V;
            if (static_cast<size_t>(nr) * nc * e <= cap || nr <= row_q) {
                const double cost = (cdiv(V, nc) - 1) * 8.0 * N * H * (need_dx ? 1 : 0) +
                                    (cdiv(N, nr) - 1) * 8.0 * V * H * (need_dw ? 1 : 0);
                if (cost < best) {
                    best = cost;
                    p.nr = nr;
                    p.nc = nc;
                }
            }
            if (nr <= row_q) break;
            // next candidate: the largest 128 * 2^k below nr
            long long next = row_q;
            while (next * 2 < nr) next *= 2;
            nr = next;
        }
    }
    p.n_rblk = N > 0 ? cdiv(N, p.nr) : 0;
    p.n_cblk = cdiv(V, p.nc);
    p.ldg = static_cast<long long>(align_up(static_cast<size_t>(p.nc), 256));
    p.bn = use_tc ? kBN : kSimtBN;
    size_t off = 0;
    p.off_count = off;
    off += 256;
    p.off_rowscale = off;
    off += align_up(static_cast<size_t>(N > 0 ? N : 1) * sizeof(float), 256);
    p.off_g = off;
    off += align_up(static_cast<size_t>(p.nr) * p.ldg * e, 256);
    p.off_dx_scratch = off;
    p.dx_slab_floats = cdiv(p.nr, 2 * kBM) * 2 * cdiv(H, p.bn) * kBM * p.bn;  // even tile count: CTA pairs
    p.dx_splits = (need_dx && p.n_cblk == 1) ? (use_tc ? choose_k_splits(p.nr, H, p.nc, cta_group_of(flags)) : choose_k_splits_simt(p.nr, H, p.nc)) : 1;
    p.dw_splits = (need_dw && p.n_rblk == 1) ? (use_tc ? choose_k_splits(p.nc, H, p.nr, cta_group_of(flags)) : choose_k_splits_simt(p.nc, H, p.nr)) : 1;
    if (need_dx && (p.n_cblk > 1 || p.dx_splits > 1))
        off += align_up(static_cast<size_t>(p.dx_splits) * p.dx_slab_floats * sizeof(float), 256);
    p.off_dw_scratch = off;
    p.dw_band_scratch_floats = cdiv(p.nc, 2 * kBM) * 2 * cdiv(H, p.bn) * kBM * p.bn;  // even tile count: CTA pairs
    if (need_dw && p.n_rblk > 1)
        off += align_up(static_cast<size_t>(p.n_cblk) * p.dw_band_scratch_floats * sizeof(float), 256);
    else if (need_dw && p.dw_splits > 1)  // slices of one band at a time
        off += align_up(static_cast<size_t>(p.dw_splits) * p.dw_band_scratch_floats * sizeof(float), 256);
    p.off_sumsq = off;
    p.sumsq_floats = cdiv(V, kBM) * cdiv(H, p.bn) * 4;
    if (need_dw) {
        const long long standalone = kSumsqBlocks;  // a split dW contraction takes the separate sum-of-squares pass
        off += align_up(static_cast<size_t>(p.sumsq_floats > standalone ? p.sumsq_floats : standalone) * sizeof(float), 256);
    }
    p.total = off;
    return p;
}

// Whether a 16-bit result may leave the tcgen05 epilogue as whole 128-byte lines (store_block64): needs 16-byte
// aligned rows. HELION_B200_EPI_WIDE=0 (tuning knob) switches back to per-thread row stores.
inline int wide_stores(const void* out, long long ld) {
    static const int kEnabled = [] { const char* e = getenv("HELION_B200_EPI_WIDE"); return e ? atoi(e) : 1; }();
    return (kEnabled != 0 && aligned16(out) && ld % 8 == 0) ? 1 : 0;
}

// HELION_B200_BWD_ONE=0 (tuning knob) keeps the dX and dW GEMMs of very small batches in separate launches.
inline bool two_products_enabled() {
    static const bool kEnabled = [] { const char* e = getenv("HELION_B200_BWD_ONE"); return e ? atoi(e) != 0 : true; }();
    return kEnabled;
}

// Small batches skip the rowscale launch: the recompute epilogue derives the per-row factor itself.
inline bool fold_rowscale(long long N) { return N <= 1024; }

int store_mode(long long idx, long long count) {
    if (count <= 1) return kStoreDirect;
    if (idx == 0) return kStoreFirst;
    return idx == count - 1 ? kStoreLast : kStoreAccum;
}

template <class T, class TDx>
int backward_impl(const DeviceInfo& d, const Path& path, const BwdPlan& p, const void* x, const void* w,
                  const void* tgt, int tgt_i64, const float* lse, long long N, long long H, long long V,
                  long long vocab_start, void* dx, void* dw, char* ws, unsigned flags, void* const* dx_events,
                  const lce_peer_scatter* scatter, float* dw_sumsq, const float* grad_out, int reduction,
                  long long ignore_index, cudaStream_t stream) {
    const bool need_dx = !(flags & LCE_FLAG_NO_DX), need_dw = !(flags & LCE_FLAG_NO_DW);
    const bool use_tc = path.use_tc;
    const int cg = path.cg;
    const T* xp = static_cast<const T*>(x);
    const T* wp = static_cast<const T*>(w);
    T* g = reinterpret_cast<T*>(ws + p.off_g);
    const float* rowscale = reinterpret_cast<const float*>(ws + p.off_rowscale);
    constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;

    for (long long rb = 0; rb < p.n_rblk; ++rb) {
        const long long r0 = rb * p.nr;
        const long long nr = (N - r0 < p.nr) ? N - r0 : p.nr;
        for (long long cb = 0; cb < p.n_cblk; ++cb) {
            const long long c0 = cb * p.nc;
            const long long nc = (V - c0 < p.nc) ? V - c0 : p.nc;
            int rc;
            // ---- step 1: G block = (softmax - onehot) * rowscale, from recomputed logits
            {
                typename EpiGrad<T>::Params ep;
                ep.tgt = tgt;
                ep.tgt_i64 = tgt_i64;
                ep.rows = static_cast<int>(nr);
                ep.cols = static_cast<int>(nc);
                ep.row_off = static_cast<int>(r0);
                ep.col_global0 = vocab_start + c0;
                ep.lse = lse;
                ep.rowscale = fold_rowscale(N) ? nullptr : rowscale;
                ep.grad_out = grad_out;
                ep.go_per_row = reduction == LCE_REDUCTION_NONE ? 1 : 0;
                ep.mean = reduction == LCE_REDUCTION_MEAN ? 1 : 0;
                ep.n_total = static_cast<int>(N);
                ep.ignore_index = ignore_index;
                ep.g = g;
                ep.ldg = p.ldg;
                ep.wide = wide_stores(g, p.ldg);
                const Mat a{xp + r0 * H, nr, H, H}, b{wp + c0 * H, nc, H, H};
                if (use_tc) {
                    if constexpr (sizeof(T) == 2)
                        rc = launch_tc<false, false, kBf16, EpiGrad<T>>(d, cg, a, b, nr, nc, H, 1, ep, stream, 1, path.sched);
                    else rc = LCE_ERR_ARG;
                } else {
                    rc = launch_simt<T, EpiGrad<T>>(d, a, false, b, false, nr, nc, H, ep, stream);
                }
                if (rc) return rc;
            }
            const Mat gm{g, nr, nc, p.ldg};
            // ---- steps 2 and 3 in one launch for a handful of tokens: dX and dW both read G and are independent
            // of each other, and at this size each is a few tiles that a launch of its own would only wait for
            bool both_done = false;
            if constexpr (sizeof(T) == 2 && std::is_same<TDx, T>::value) {
                if (use_tc && need_dx && need_dw && N <= 128 && p.n_rblk == 1 && p.n_cblk == 1 && scatter == nullptr &&
                    dx_events == nullptr && dw_sumsq == nullptr && two_products_enabled()) {
                    typename EpiStore<T>::Params e1, e2;
                    e1.out = static_cast<T*>(dx);
                    e1.ldo = H;
                    e1.rows = static_cast<int>(nr);
                    e1.cols = static_cast<int>(H);
                    e1.scratch = reinterpret_cast<float*>(ws + p.off_dx_scratch);
                    e1.mode = p.dx_splits > 1 ? kStoreSlice : kStoreDirect;
                    e1.slab_floats = p.dx_slab_floats;
                    e1.peer_world = 0;
                    e1.wide = wide_stores(e1.out, H);
                    e2.out = static_cast<T*>(dw);
                    e2.ldo = H;
                    e2.rows = static_cast<int>(nc);
                    e2.cols = static_cast<int>(H);
                    e2.scratch = reinterpret_cast<float*>(ws + p.off_dw_scratch);
                    e2.mode = p.dw_splits > 1 ? kStoreSlice : kStoreDirect;
                    e2.slab_floats = p.dw_band_scratch_floats;
                    e2.peer_world = 0;
                    e2.wide = wide_stores(e2.out, H);
                    const GemmProblem q1{gm, Mat{wp, nc, H, H}, nr, H, nc, p.dx_splits};
                    const GemmProblem q2{gm, Mat{xp, nr, H, H}, nc, H, nr, p.dw_splits};
                    if ((rc = launch_tc_two<kBf16, EpiStore<T>>(d, q1, e1, q2, e2, stream))) return rc;
                    const int bn = static_cast<int>(p.bn);
                    const int n_tiles = static_cast<int>(cdiv(H, bn));
                    auto sum_slices = [&](const typename EpiStore<T>::Params& e, int splits, long long rows) -> int {
                        if (splits <= 1) return LCE_OK;
                        const int m_tiles = static_cast<int>(cdiv(rows, kBM));
                        const long long quads = static_cast<long long>(m_tiles) * n_tiles * (bn / 4) * kBM;
                        const int blocks = static_cast<int>(cdiv(quads, 256) < 4096 ? cdiv(quads, 256) : 4096);
                        const cudaError_t err = launch_dependent(
                            splitk_reduce_kernel<T>, blocks, 256, stream, static_cast<const float*>(e.scratch), splits,
                            e.slab_floats, m_tiles, n_tiles, bn, static_cast<int>(rows), static_cast<int>(H), e.out, H);
                        LCE_COUNT_LAUNCH();
                        return cuda_failed(err) ? LCE_ERR_CUDA : LCE_OK;
                    };
                    if ((rc = sum_slices(e1, p.dx_splits, nr))) return rc;
                    if ((rc = sum_slices(e2, p.dw_splits, nc))) return rc;
                    both_done = true;
                }
            }
            if (both_done) continue;
            // ---- step 2: dX[r0 : r0+nr, :] (+)= G @ W[c0 : c0+nc, :]
            if (need_dx) {
                typename EpiStore<TDx>::Params ep;
                ep.out = static_cast<TDx*>(dx) + r0 * H;
                ep.ldo = H;
                ep.rows = static_cast<int>(nr);
                ep.cols = static_cast<int>(H);
                ep.scratch = reinterpret_cast<float*>(ws + p.off_dx_scratch);
                ep.mode = store_mode(cb, p.n_cblk);
                ep.slab_floats = p.dx_slab_floats;
                ep.peer_world = 0;
                ep.wide = wide_stores(ep.out, H);
                if constexpr (std::is_same<TDx, float>::value) {
                    if (scatter != nullptr) {  // finished rows go straight to the GPUs that own them
                        ep.peer_world = scatter->world;
                        ep.peer_rank = scatter->rank;
                        ep.rows_per_rank = static_cast<int>(cdiv(N, scatter->world));
                        ep.row_off = static_cast<int>(r0);
                        for (int k = 0; k < scatter->world; ++k) ep.peer[k] = static_cast<float*>(scatter->staging[k]);
                        ep.out = nullptr;
                    }
                }
                const Mat b{wp + c0 * H, nc, H, H};
                // few output tiles (short row chunk): cut the vocabulary contraction into slices
                const int splits = (p.dx_splits > 1 && nr == p.nr && scatter == nullptr) ? p.dx_splits : 1;
                if (splits > 1) ep.mode = kStoreSlice;
                if (use_tc) {
                    if constexpr (sizeof(T) == 2)
                        rc = launch_tc<false, true, kBf16, EpiStore<TDx>>(d, cg, gm, b, nr, H, nc, 0, ep, stream, splits, path.sched);
                    else rc = LCE_ERR_ARG;
                } else {
                    rc = launch_simt<T, EpiStore<TDx>>(d, gm, false, b, true, nr, H, nc, ep, stream, splits);
                }
                if (rc) return rc;
                if (splits > 1) {
                    const int bn = static_cast<int>(p.bn);
                    const int m_tiles = static_cast<int>(cdiv(nr, kBM)), n_tiles = static_cast<int>(cdiv(H, bn));
                    const long long quads = static_cast<long long>(m_tiles) * n_tiles * (bn / 4) * kBM;
                    const int blocks = static_cast<int>(cdiv(quads, 256) < 4096 ? cdiv(quads, 256) : 4096);
                    const cudaError_t err = launch_dependent(
                        splitk_reduce_kernel<TDx>, blocks, 256, stream, static_cast<const float*>(ep.scratch), splits,
                        p.dx_slab_floats, m_tiles, n_tiles, bn, static_cast<int>(nr), static_cast<int>(H), ep.out, H);
                    LCE_COUNT_LAUNCH();
                    if (cuda_failed(err)) return LCE_ERR_CUDA;
                }
                // rows r0.. of dX are final after the last band: let the caller start reducing them
                // while the dW GEMM below (and later chunks) still run
                if (dx_events && cb == p.n_cblk - 1 && dx_events[rb] &&
                    cudaEventRecord(static_cast<cudaEvent_t>(dx_events[rb]), stream) != cudaSuccess)
                    return LCE_ERR_CUDA;
            }
            // ---- step 3: dW[c0 : c0+nc, :] (+)= G^T @ X[r0 : r0+nr, :]
            if (need_dw) {
                typename EpiStore<T>::Params ep;
                ep.out = static_cast<T*>(dw) + c0 * H;
                ep.ldo = H;
                ep.rows = static_cast<int>(nc);
                ep.cols = static_cast<int>(H);
                ep.scratch = reinterpret_cast<float*>(ws + p.off_dw_scratch) + cb * p.dw_band_scratch_floats;
                ep.mode = store_mode(rb, p.n_rblk);
                ep.slab_floats = p.dw_band_scratch_floats;
                ep.peer_world = 0;
                ep.wide = wide_stores(ep.out, H);
                if (dw_sumsq != nullptr && p.dw_splits == 1) {  // gradient-norm partials ride on the final stores
                    ep.sumsq_partial = reinterpret_cast<float*>(ws + p.off_sumsq);
                    ep.sumsq_tile0 = static_cast<int>(c0 / kBM);
                }
                const Mat b{xp + r0 * H, nr, H, H};
                // short vocabulary block (few output tiles): cut the token contraction into slices
                const int wsplits = (p.dw_splits > 1 && p.n_rblk == 1 && nc == p.nc) ? p.dw_splits : 1;
                if (wsplits > 1) {
                    ep.mode = kStoreSlice;
                    ep.scratch = reinterpret_cast<float*>(ws + p.off_dw_scratch);
                }
                if (use_tc) {
                    if constexpr (sizeof(T) == 2)
                        rc = launch_tc<true, true, kBf16, EpiStore<T>>(d, cg, gm, b, nc, H, nr, 0, ep, stream, wsplits, path.sched);
                    else rc = LCE_ERR_ARG;
                } else {
                    rc = launch_simt<T, EpiStore<T>>(d, gm, true, b, true, nc, H, nr, ep, stream, wsplits);
                }
                if (rc) return rc;
                if (wsplits > 1) {
                    const int bn = static_cast<int>(p.bn);
                    const int m_tiles = static_cast<int>(cdiv(nc, kBM)), n_tiles = static_cast<int>(cdiv(H, bn));
                    const long long quads = static_cast<long long>(m_tiles) * n_tiles * (bn / 4) * kBM;
                    const int blocks = static_cast<int>(cdiv(quads, 256) < 4096 ? cdiv(quads, 256) : 4096);
                    const cudaError_t err = launch_dependent(
                        splitk_reduce_kernel<T>, blocks, 256, stream, static_cast<const float*>(ep.scratch), wsplits,
                        p.dw_band_scratch_floats, m_tiles, n_tiles, bn, static_cast<int>(nc), static_cast<int>(H), ep.out, H);
                    LCE_COUNT_LAUNCH();
                    if (cuda_failed(err)) return LCE_ERR_CUDA;
                }
            }
        }
    }
    if (dw_sumsq != nullptr && need_dw) {
        float* partials = reinterpret_cast<float*>(ws + p.off_sumsq);
        int count = static_cast<int>(p.sumsq_floats);
        if (p.dw_splits > 1) {  // dW came out of the split-K reduction: one read of it, as lce_sumsq does
            sumsq_partial_kernel<T><<<kSumsqBlocks, kOptThreads, 0, stream>>>(static_cast<const T*>(dw), V * H, partials);
            LCE_COUNT_LAUNCH();
            if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
            count = kSumsqBlocks;
        }
        sumsq_final_kernel<<<1, 1024, 0, stream>>>(partials, count, dw_sumsq, 0);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    return LCE_OK;
}

}  // namespace
}  // namespace lce

using namespace lce;

extern "C" {

int lce_version(void) { return LCE_VERSION; }

unsigned long long lce_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* lce_last_cuda_error(void) { return cudaGetErrorName(t_last_cuda_error); }

void lce_set_tuning(int band_mb, int l2_hint_mode, int dyn_waves) {
    if (band_mb > 0) g_tuning.band_mb.store(band_mb, std::memory_order_relaxed);
    if (l2_hint_mode >= 0) g_tuning.hint_mode.store(l2_hint_mode, std::memory_order_relaxed);
    if (dyn_waves >= 0) g_tuning.dyn_waves.store(dyn_waves, std::memory_order_relaxed);
}

const char* lce_strerror(int code) {
    switch (code) {
        case LCE_OK: return "ok";
        case LCE_ERR_ARG: return "invalid argument (null pointer, bad size or unknown enum)";
        case LCE_ERR_ALIGN: return "tcgen05 path needs 16-byte aligned pointers and hidden_size % 8 == 0";
        case LCE_ERR_WS_TOO_SMALL: return "workspace too small";
        case LCE_ERR_ARCH: return "device is not compute capability 10.x (sm_100a only, no fallback)";
        case LCE_ERR_CUDA: return "CUDA runtime or driver call failed";
        case LCE_ERR_TOO_LARGE: return "dimension too large for 32-bit tile indexing";
        case LCE_ERR_STATIC_SCRATCH:
            return "problem needs more than the 16 MiB of built-in scratch; use lce_forward_stats with a workspace";
        default: return "unknown error";
    }
}

int lce_device_status(int* status_out, int clear) {
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    if (cudaDeviceSynchronize() != cudaSuccess) return LCE_ERR_CUDA;
    int v = 0;
    if (cudaMemcpy(&v, d->status_ptr, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return LCE_ERR_CUDA;
    if (clear && v != 0) {
        const int zero = 0;
        if (cudaMemcpy(d->status_ptr, &zero, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess) return LCE_ERR_CUDA;
    }
    if (status_out) *status_out = v;
    return LCE_OK;
}

size_t lce_forward_workspace_bytes(int64_t N, int64_t H, int64_t V, int dtype, unsigned flags) {
    if (check_dims(N, H, V, dtype)) return 0;
    // size for the finer (SIMT) tiling unless the caller pins the tcgen05 path
    const bool tc_only = (flags & LCE_FLAG_FORCE_TC) != 0;
    return align_up(fwd_layout(N, V, tc_only).bytes, 256) + 256;
}

int lce_forward_stats(const void* x, const void* w, const void* target, int target_is_i64, int64_t N,
                      int64_t H, int64_t V, int64_t vocab_start, int dtype, float* stats, void* ws,
                      size_t ws_bytes, unsigned flags, void* stream) {
    int rc = check_dims(N, H, V, dtype);
    if (rc) return rc;
    if (N == 0) return LCE_OK;
    if (!x || !w || !target || !stats || !ws) return LCE_ERR_ARG;
    DeviceInfo* d;
    if ((rc = device_info(&d))) return rc;
    bool use_tc;
    if ((rc = choose_path(dtype, H, x, w, flags, &use_tc))) return rc;
    if (ws_bytes < fwd_layout(N, V, use_tc).bytes) return LCE_ERR_WS_TOO_SMALL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    FwdOutputs fo;
    fo.stats = stats;
    const size_t sched_off = align_up(fwd_layout(N, V, use_tc).bytes, 256);  // the slack lce_forward_workspace_bytes adds
    const Path path{use_tc, cta_group_of(flags),
                    ws_bytes >= sched_off + sizeof(int) ? reinterpret_cast<int*>(static_cast<char*>(ws) + sched_off) : nullptr};
    switch (dtype) {
        case LCE_DTYPE_BF16:
            return forward_stats_impl<__nv_bfloat16>(*d, path, x, w, target, target_is_i64, N, H, V, vocab_start, fo, ws, s);
        case LCE_DTYPE_F16:
            return forward_stats_impl<__half>(*d, path, x, w, target, target_is_i64, N, H, V, vocab_start, fo, ws, s);
        default:
            return forward_stats_impl<float>(*d, path, x, w, target, target_is_i64, N, H, V, vocab_start, fo, ws, s);
    }
}

int lce_greedy_head(const void* x, const void* w, int64_t N, int64_t H, int64_t V, int64_t vocab_start, int dtype,
                    int64_t* token, float* logprob, float* lse, void* ws, size_t ws_bytes, unsigned flags,
                    void* stream) {
    int rc = check_dims(N, H, V, dtype);
    if (rc) return rc;
    if (N == 0) return LCE_OK;
    if (!x || !w || !token || !logprob || !ws) return LCE_ERR_ARG;
    DeviceInfo* d;
    if ((rc = device_info(&d))) return rc;
    bool use_tc;
    if ((rc = choose_path(dtype, H, x, w, flags, &use_tc))) return rc;
    if (ws_bytes < fwd_layout(N, V, use_tc).bytes) return LCE_ERR_WS_TOO_SMALL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    long long* tok = reinterpret_cast<long long*>(token);
    const size_t sched_off = align_up(fwd_layout(N, V, use_tc).bytes, 256);
    const Path path{use_tc, cta_group_of(flags),
                    ws_bytes >= sched_off + sizeof(int) ? reinterpret_cast<int*>(static_cast<char*>(ws) + sched_off) : nullptr};
    switch (dtype) {
        case LCE_DTYPE_BF16:
            return greedy_head_impl<__nv_bfloat16>(*d, path, x, w, N, H, V, vocab_start, tok, logprob, lse, ws, s);
        case LCE_DTYPE_F16:
            return greedy_head_impl<__half>(*d, path, x, w, N, H, V, vocab_start, tok, logprob, lse, ws, s);
        default:
            return greedy_head_impl<float>(*d, path, x, w, N, H, V, vocab_start, tok, logprob, lse, ws, s);
    }
}

size_t lce_topk_workspace_bytes(int64_t N, int64_t H, int64_t V, int dtype, unsigned flags) {
    if (check_dims(N, H, V, dtype)) return 0;
    const bool tc_only = (flags & LCE_FLAG_FORCE_TC) != 0;  // else sized for the finer CUDA-core tiling
    return align_up(topk_partial_bytes(N, V, tc_only), 256) + 256;
}

int lce_topk_head(const void* x, const void* w, int64_t N, int64_t H, int64_t V, int64_t vocab_start, int dtype,
                  int k, float inv_temperature, float* top_val, int64_t* top_idx, float* lse, void* ws,
                  size_t ws_bytes, unsigned flags, void* stream) {
    int rc = check_dims(N, H, V, dtype);
    if (rc) return rc;
    if (k < 1 || k > kTopkMaxK || !(inv_temperature > 0.f)) return LCE_ERR_ARG;
    if (N == 0) return LCE_OK;
    if (!x || !w || !top_val || !top_idx || !lse || !ws) return LCE_ERR_ARG;
    DeviceInfo* d;
    if ((rc = device_info(&d))) return rc;
    bool use_tc;
    if ((rc = choose_path(dtype, H, x, w, flags, &use_tc))) return rc;
    const size_t partial = topk_partial_bytes(N, V, use_tc);
    if (ws_bytes < partial) return LCE_ERR_WS_TOO_SMALL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t sched_off = align_up(partial, 256);
    const Path path{use_tc, cta_group_of(flags),
                    ws_bytes >= sched_off + sizeof(int) ? reinterpret_cast<int*>(static_cast<char*>(ws) + sched_off) : nullptr};
    long long* idx = reinterpret_cast<long long*>(top_idx);
    switch (dtype) {
        case LCE_DTYPE_BF16:
            return topk_head_impl<__nv_bfloat16>(*d, path, x, w, N, H, V, vocab_start, k, inv_temperature, top_val, idx, lse, ws, s);
        case LCE_DTYPE_F16:
            return topk_head_impl<__half>(*d, path, x, w, N, H, V, vocab_start, k, inv_temperature, top_val, idx, lse, ws, s);
        default:
            return topk_head_impl<float>(*d, path, x, w, N, H, V, vocab_start, k, inv_temperature, top_val, idx, lse, ws, s);
    }
}

size_t lce_finalize_workspace_bytes(int64_t N) {
    return align_up(static_cast<size_t>(N > 0 ? N : 1) * sizeof(float), 256);
}

int lce_finalize(const float* stats, int R, const void* target, int target_is_i64, int64_t N,
                 int64_t ignore_index, int reduction, float* lse, float* loss, float* valid_count,
                 void* ws, size_t ws_bytes, void* stream) {
    if (N < 0 || R < 1 || N > 0x7fffff00ll) return LCE_ERR_ARG;
    if (reduction != LCE_REDUCTION_NONE && reduction != LCE_REDUCTION_MEAN && reduction != LCE_REDUCTION_SUM)
        return LCE_ERR_ARG;
    if (!loss) return LCE_ERR_ARG;
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* loss_rows = reduction == LCE_REDUCTION_NONE ? loss : static_cast<float*>(ws);
    if (N > 0) {
        if (!stats || !target || !lse) return LCE_ERR_ARG;
        if (reduction != LCE_REDUCTION_NONE && (!ws || ws_bytes < static_cast<size_t>(N) * sizeof(float)))
            return LCE_ERR_WS_TOO_SMALL;
        const int threads = 256;
        finalize_rows_kernel<<<static_cast<int>(cdiv(N, threads)), threads, 0, s>>>(
            stats, R, target, target_is_i64, static_cast<int>(N), ignore_index, lse, loss_rows);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    if (reduction != LCE_REDUCTION_NONE || valid_count) {
        reduce_loss_kernel<<<1, 1024, 0, s>>>(loss_rows, target, target_is_i64, static_cast<int>(N), ignore_index,
                                              reduction == LCE_REDUCTION_MEAN ? 1 : 0,
                                              reduction == LCE_REDUCTION_NONE ? nullptr : loss, valid_count);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    return LCE_OK;
}

size_t lce_forward_loss_workspace_bytes(int64_t N, int64_t H, int64_t V, int dtype, unsigned flags) {
    const size_t partial = lce_forward_workspace_bytes(N, H, V, dtype, flags);
    return partial ? partial + lce_finalize_workspace_bytes(N) : 0;
}

int lce_forward_loss(const void* x, const void* w, const void* target, int target_is_i64, int64_t N, int64_t H,
                     int64_t V, int dtype, int64_t ignore_index, int reduction, float* lse, float* loss,
                     float* valid_count, void* ws, size_t ws_bytes, unsigned flags, void* stream) {
    int rc = check_dims(N, H, V, dtype);
    if (rc) return rc;
    if (reduction != LCE_REDUCTION_NONE && reduction != LCE_REDUCTION_MEAN && reduction != LCE_REDUCTION_SUM)
        return LCE_ERR_ARG;
    if (N == 0) return LCE_ERR_ARG;  // the empty batch is the caller's business (zero loss, no launch)
    if (!x || !w || !target || !lse || !loss || !ws) return LCE_ERR_ARG;
    DeviceInfo* d;
    if ((rc = device_info(&d))) return rc;
    bool use_tc;
    if ((rc = choose_path(dtype, H, x, w, flags, &use_tc))) return rc;
    const size_t partial_bytes = align_up(fwd_layout(N, V, use_tc).bytes, 256);
    if (ws_bytes < partial_bytes + static_cast<size_t>(N) * sizeof(float)) return LCE_ERR_WS_TOO_SMALL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    FwdOutputs fo;
    fo.lse = lse;
    fo.loss_rows = reduction == LCE_REDUCTION_NONE ? loss : reinterpret_cast<float*>(static_cast<char*>(ws) + partial_bytes);
    fo.ignore_index = ignore_index;
    // few rows and few vocabulary tiles: one CTA finishes the whole forward after the GEMM, as long as each of
    // its threads folds at most 16 tiles (1024 threads = roundup(N, 32) row lanes x tile lanes)
    {
        const long long row_lanes = cdiv(N, 32) * 32;
        const long long tile_lanes = row_lanes <= 1024 ? (1024 / row_lanes < 32 ? 1024 / row_lanes : 32) : 0;
        fo.one_launch_tail = tile_lanes > 0 && cdiv(fwd_layout(N, V, use_tc).n_tiles, tile_lanes) <= 16;
    }
    fo.reduction = reduction;
    fo.loss = loss;
    fo.valid_count = valid_count;
    const size_t sched_off = partial_bytes + align_up(static_cast<size_t>(N) * sizeof(float), 256);
    const Path path{use_tc, cta_group_of(flags),
                    ws_bytes >= sched_off + sizeof(int) ? reinterpret_cast<int*>(static_cast<char*>(ws) + sched_off) : nullptr};
    switch (dtype) {
        case LCE_DTYPE_BF16:
            rc = forward_stats_impl<__nv_bfloat16>(*d, path, x, w, target, target_is_i64, N, H, V, 0, fo, ws, s);
            break;
        case LCE_DTYPE_F16:
            rc = forward_stats_impl<__half>(*d, path, x, w, target, target_is_i64, N, H, V, 0, fo, ws, s);
            break;
        default:
            rc = forward_stats_impl<float>(*d, path, x, w, target, target_is_i64, N, H, V, 0, fo, ws, s);
    }
    if (rc) return rc;
    if (!fo.one_launch_tail && (reduction != LCE_REDUCTION_NONE || valid_count)) {
        reduce_loss_kernel<<<1, 1024, 0, s>>>(fo.loss_rows, target, target_is_i64, static_cast<int>(N), ignore_index,
                                              reduction == LCE_REDUCTION_MEAN ? 1 : 0,
                                              reduction == LCE_REDUCTION_NONE ? nullptr : loss, valid_count);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    return LCE_OK;
}

size_t lce_backward_workspace_bytes(int64_t N, int64_t H, int64_t V, int dtype, unsigned flags,
                                    size_t block_bytes) {
    if (check_dims(N, H, V, dtype)) return 0;
    // the SIMT and tcgen05 plans differ only in scratch tiling; report the larger of the two
    const size_t a = plan_backward(N, H, V, dtype, true, flags, block_bytes).total;
    const size_t b = plan_backward(N, H, V, dtype, false, flags, block_bytes).total;
    return a > b ? a : b;
}

int lce_backward_plan(int64_t N, int64_t H, int64_t V, int dtype, unsigned flags, size_t block_bytes,
                      const void* x, const void* w, int64_t* out) {
    int rc = check_dims(N, H, V, dtype);
    if (rc) return rc;
    if (!out) return LCE_ERR_ARG;
    bool use_tc;
    if ((rc = choose_path(dtype, H, x, w, flags, &use_tc))) return rc;
    const BwdPlan p = plan_backward(N, H, V, dtype, use_tc, flags, block_bytes);
    out[0] = p.nr;
    out[1] = p.nc;
    out[2] = p.n_rblk;
    out[3] = p.n_cblk;
    return LCE_OK;
}

int lce_backward(const void* x, const void* w, const void* target, int target_is_i64, const float* lse,
                 const float* grad_out, int64_t N, int64_t H, int64_t V, int64_t vocab_start, int dtype,
                 int64_t ignore_index, int reduction, void* dx, void* dw, void* ws, size_t ws_bytes,
                 unsigned flags, size_t block_bytes, void* const* dx_events, const lce_peer_scatter* scatter,
                 float* dw_sumsq, void* stream) {
    int rc = check_dims(N, H, V, dtype);
    if (rc) return rc;
    if (reduction != LCE_REDUCTION_NONE && reduction != LCE_REDUCTION_MEAN && reduction != LCE_REDUCTION_SUM)
        return LCE_ERR_ARG;
    const bool need_dx = !(flags & LCE_FLAG_NO_DX), need_dw = !(flags & LCE_FLAG_NO_DW);
    if (scatter != nullptr) {
        if (!(flags & LCE_FLAG_DX_F32) || scatter->world < 1 || scatter->world > kMaxPeers || scatter->rank < 0 ||
            scatter->rank >= scatter->world || (H % 4) != 0)
            return LCE_ERR_ARG;
        for (int k = 0; k < scatter->world; ++k)
            if (!scatter->staging[k] || !aligned16(scatter->staging[k])) return LCE_ERR_ARG;
    }
    if ((need_dx && !dx && !scatter && N > 0) || (need_dw && !dw)) return LCE_ERR_ARG;
    if (dw_sumsq && need_dw && !aligned16(dw)) return LCE_ERR_ALIGN;
    DeviceInfo* d;
    if ((rc = device_info(&d))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N == 0) {
        // no rows: dW is all zeros (tritium/ops/cross_entropy.py:912-913), dX is empty
        if (need_dw && cudaMemsetAsync(dw, 0, static_cast<size_t>(V) * H * elem_size(dtype), s) != cudaSuccess)
            return LCE_ERR_CUDA;
        if (need_dw && dw_sumsq && cudaMemsetAsync(dw_sumsq, 0, sizeof(float), s) != cudaSuccess) return LCE_ERR_CUDA;
        return LCE_OK;
    }
    if (!x || !w || !target || !lse || !grad_out || !ws) return LCE_ERR_ARG;
    if (!need_dx && !need_dw) return LCE_OK;
    bool use_tc;
    if ((rc = choose_path(dtype, H, x, w, flags, &use_tc))) return rc;
    const BwdPlan p = plan_backward(N, H, V, dtype, use_tc, flags, block_bytes);
    if (ws_bytes < p.total) return LCE_ERR_WS_TOO_SMALL;
    char* wsc = static_cast<char*>(ws);
    float* count = reinterpret_cast<float*>(wsc + p.off_count);
    float* rowscale = reinterpret_cast<float*>(wsc + p.off_rowscale);
    // small batches count their valid rows inside the rowscale launch; large ones in a launch of its own
    const bool separate_count = reduction == LCE_REDUCTION_MEAN && N > 16384;
    if (separate_count) {
        count_valid_kernel<<<1, 1024, 0, s>>>(target, target_is_i64, static_cast<int>(N), ignore_index, count);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    if (!fold_rowscale(N)) {
        rowscale_kernel<<<static_cast<int>(cdiv(N, 256)), 256, 0, s>>>(
            target, target_is_i64, static_cast<int>(N), ignore_index, grad_out,
            reduction == LCE_REDUCTION_NONE ? 1 : 0, reduction == LCE_REDUCTION_MEAN ? 1 : 0,
            separate_count ? count : nullptr, rowscale);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    const bool dx32 = (flags & LCE_FLAG_DX_F32) != 0;
    // the 256-byte head of the workspace holds the valid-row count (float 0) and the tile-deal counter (byte 128)
    const Path path{use_tc, cta_group_of(flags), reinterpret_cast<int*>(wsc + p.off_count + 128)};
#define LCE_BWD(T)                                                                                          \
    (dx32 ? backward_impl<T, float>(*d, path, p, x, w, target, target_is_i64, lse, N, H, V, vocab_start, \
                                    dx, dw, wsc, flags, dx_events, scatter, dw_sumsq, grad_out, reduction,     \
                                    ignore_index, s)                                                        \
          : backward_impl<T, T>(*d, path, p, x, w, target, target_is_i64, lse, N, H, V, vocab_start, dx, \
                                dw, wsc, flags, dx_events, nullptr, dw_sumsq, grad_out, reduction, ignore_index, s))
    switch (dtype) {
        case LCE_DTYPE_BF16: return LCE_BWD(__nv_bfloat16);
        case LCE_DTYPE_F16: return LCE_BWD(__half);
        default: return LCE_BWD(float);
    }
#undef LCE_BWD
}

int lce_debug_wait_test(unsigned long long limit_ns, unsigned announce_extra_bytes) {
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    const unsigned long long limit = limit_ns ? limit_ns : LCE_WAIT_LIMIT_NS;
    if (cudaDeviceSynchronize() != cudaSuccess) return LCE_ERR_CUDA;
    if (cudaMemcpyToSymbol(ptx::g_wait_limit_ns, &limit, sizeof(limit)) != cudaSuccess) return LCE_ERR_CUDA;
    if (cudaMemcpyToSymbol(ptx::g_debug_announce_extra, &announce_extra_bytes, sizeof(unsigned)) != cudaSuccess)
        return LCE_ERR_CUDA;
    return LCE_OK;
}

int lce_debug_gemm(const void* a, const void* b, float* out, int64_t M, int64_t N, int64_t K,
                   int a_mn, int b_mn, int dtype, unsigned flags, void* stream) {
    if (!a || !b || !out || M <= 0 || N <= 0 || K <= 0) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16) return LCE_ERR_ARG;
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int cg = cta_group_of(flags);
    EpiStore<float>::Params ep;
    ep.out = out;
    ep.ldo = N;
    ep.rows = static_cast<int>(M);
    ep.cols = static_cast<int>(N);
    ep.scratch = nullptr;
    ep.mode = kStoreDirect;
    ep.slab_floats = 0;
    ep.peer_world = 0;
    const Mat am = a_mn ? Mat{a, K, M, M} : Mat{a, M, K, K};
    const Mat bm = b_mn ? Mat{b, K, N, N} : Mat{b, N, K, K};
#define LCE_DBG(AMN, BMN)                                                                               \
    (dtype == LCE_DTYPE_BF16 ? launch_tc<AMN, BMN, true, EpiStore<float>>(*d, cg, am, bm, M, N, K, 1, ep, s) \
                             : launch_tc<AMN, BMN, false, EpiStore<float>>(*d, cg, am, bm, M, N, K, 1, ep, s))
    if (!a_mn && !b_mn) return LCE_DBG(false, false);
    if (!a_mn && b_mn) return LCE_DBG(false, true);
    if (a_mn && !b_mn) return LCE_DBG(true, false);
    return LCE_DBG(true, true);
#undef LCE_DBG
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Forward statistics with library-owned scratch (no allocation by anyone at call time)
// ---------------------------------------------------------------------------------------------
namespace lce {
namespace {

// Scratch for the per-(vocab tile, row) partial statistics of lce_forward_stats_static. It is part
// of the library image: every GPU that loads the library carries these 16 MiB until the process
// exits. In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
constexpr size_t kStaticScratchBytes = 16ull << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

void* g_static_scratch_ptr[kMaxDevices] = {};

// Resolves the device address of g_static_scratch once per device (the device must be current).
int static_scratch_address(void** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return LCE_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return LCE_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return LCE_ERR_CUDA;
        g_static_scratch_ptr[dev] = p;
    }
    *out = g_static_scratch_ptr[dev];
    return LCE_OK;
}

}  // namespace
}  // namespace lce

extern "C" {

size_t lce_forward_stats_static_capacity(void) { return lce::kStaticScratchBytes; }

int lce_forward_stats_static(const void* x, const void* w, const void* target, int target_is_i64, int64_t N,
                             int64_t H, int64_t V, int64_t vocab_start, int dtype, float* stats, unsigned flags,
                             void* stream) {
    int rc = check_dims(N, H, V, dtype);
    if (rc) return rc;
    if (N == 0) return LCE_OK;
    if (!x || !w || !target || !stats) return LCE_ERR_ARG;
    DeviceInfo* d;
    if ((rc = device_info(&d))) return rc;
    bool use_tc;
    if ((rc = choose_path(dtype, H, x, w, flags, &use_tc))) return rc;
    if (fwd_layout(N, V, use_tc).bytes > kStaticScratchBytes) return LCE_ERR_STATIC_SCRATCH;
    void* scratch = nullptr;
    if ((rc = static_scratch_address(&scratch))) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    FwdOutputs fo;
    fo.stats = stats;
    // Nothing in the scratch has to start at zero: the GEMM epilogue writes every (tile, row) entry
    // the merge kernel reads, earlier in this same call and on the same stream.
    switch (dtype) {
        case LCE_DTYPE_BF16:
            return forward_stats_impl<__nv_bfloat16>(*d, Path{use_tc, cta_group_of(flags)}, x, w, target, target_is_i64, N, H, V, vocab_start, fo, scratch, s);
        case LCE_DTYPE_F16:
            return forward_stats_impl<__half>(*d, Path{use_tc, cta_group_of(flags)}, x, w, target, target_is_i64, N, H, V, vocab_start, fo, scratch, s);
        default:
            return forward_stats_impl<float>(*d, Path{use_tc, cta_group_of(flags)}, x, w, target, target_is_i64, N, H, V, vocab_start, fo, scratch, s);
    }
}

}  // extern "C"

extern "C" int lce_dx_reduce_gather(const void* staging, int world, int rank, int64_t N, int64_t H, int dtype,
                                    void* const* out_ptrs, void* stream) {
    if (!staging || !out_ptrs || world < 1 || world > kMaxPeers || rank < 0 || rank >= world || N <= 0 || H <= 0 ||
        (H % 4) != 0)
        return LCE_ERR_ARG;
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    const long long rpr = cdiv(N, world);
    const long long row0 = rpr * rank;
    const long long n_rows = row0 >= N ? 0 : (N - row0 < rpr ? N - row0 : rpr);
    if (n_rows == 0) return LCE_OK;
    PeerOutputs outs;
    for (int k = 0; k < world; ++k) {
        if (!out_ptrs[k]) return LCE_ERR_ARG;
        outs.out[k] = out_ptrs[k];
    }
    const long long quads = n_rows * (H / 4);
    const int blocks = static_cast<int>(cdiv(quads, 256) < 148 * 16 ? cdiv(quads, 256) : 148 * 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float* st = static_cast<const float*>(staging);
    switch (dtype) {
        case LCE_DTYPE_BF16: dx_reduce_gather_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(st, world, rpr, H, row0, n_rows, outs); break;
        case LCE_DTYPE_F16: dx_reduce_gather_kernel<__half><<<blocks, 256, 0, s>>>(st, world, rpr, H, row0, n_rows, outs); break;
        case LCE_DTYPE_F32: dx_reduce_gather_kernel<float><<<blocks, 256, 0, s>>>(st, world, rpr, H, row0, n_rows, outs); break;
        default: return LCE_ERR_ARG;
    }
    LCE_COUNT_LAUNCH();
    return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
}

extern "C" int lce_dx_reduce_slice(const void* staging, int world, int rank, int64_t N, int64_t H, int dtype,
                                   void* out, void* stream) {
    if (!staging || !out || world < 1 || world > kMaxPeers || rank < 0 || rank >= world || N <= 0 || H <= 0 ||
        (H % 4) != 0 || !aligned16(staging) || !aligned16(out))
        return LCE_ERR_ARG;
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    const long long rpr = cdiv(N, world);
    const long long row0 = rpr * rank;
    const long long n_rows = row0 >= N ? 0 : (N - row0 < rpr ? N - row0 : rpr);
    if (n_rows == 0) return LCE_OK;
    const long long quads = n_rows * (H / 4);
    const int blocks = static_cast<int>(cdiv(quads, 256) < 148 * 16 ? cdiv(quads, 256) : 148 * 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float* st = static_cast<const float*>(staging);
    switch (dtype) {
        case LCE_DTYPE_BF16: dx_reduce_slice_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(st, world, rpr, H, n_rows, static_cast<__nv_bfloat16*>(out)); break;
        case LCE_DTYPE_F16: dx_reduce_slice_kernel<__half><<<blocks, 256, 0, s>>>(st, world, rpr, H, n_rows, static_cast<__half*>(out)); break;
        case LCE_DTYPE_F32: dx_reduce_slice_kernel<float><<<blocks, 256, 0, s>>>(st, world, rpr, H, n_rows, static_cast<float*>(out)); break;
        default: return LCE_ERR_ARG;
    }
    LCE_COUNT_LAUNCH();
    return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
}

// ---------------------------------------------------------------------------------------------
// Cross-entropy on materialised logits
// ---------------------------------------------------------------------------------------------
namespace lce {
namespace {

struct CeLayout {
    long long n_chunks, n_groups, row_stride;
    size_t off_partial, off_loss_rows, off_rowscale, off_count, total;
};

long long ce_chunk(int dtype) { return dtype == LCE_DTYPE_F32 ? CeTile<float>::kChunk : CeTile<__half>::kChunk; }

CeLayout ce_layout(long long N, long long V, int dtype) {
    CeLayout l;
    l.n_chunks = cdiv(V, ce_chunk(dtype));
    l.n_groups = cdiv(l.n_chunks, kCeChunksPerCta);  // forward CTAs per row
    l.row_stride = static_cast<long long>(align_up(static_cast<size_t>(N > 0 ? N : 1), 64));
    size_t off = 0;
    l.off_partial = off;
    off += align_up(static_cast<size_t>(l.n_groups) * 3 * l.row_stride * sizeof(float), 256);
    l.off_loss_rows = off;
    off += align_up(static_cast<size_t>(l.row_stride) * sizeof(float), 256);
    l.off_rowscale = off;
    off += align_up(static_cast<size_t>(l.row_stride) * sizeof(float), 256);
    l.off_count = off;
    off += 256;
    l.total = off;
    return l;
}

template <class T>
int ce_forward_impl(const void* logits, const void* tgt, int tgt_i64, long long N, long long V, long long ignore_index,
                    const CeLayout& l, char* ws, float* lse, float* loss_rows, cudaStream_t s) {
    const T* z = static_cast<const T*>(logits);
    const bool vec = aligned16(logits) && (V * sizeof(T)) % 16 == 0;
    float* partial = reinterpret_cast<float*>(ws + l.off_partial);
    const int grid = static_cast<int>(N * l.n_groups);
    const int nc = static_cast<int>(l.n_chunks), ng = static_cast<int>(l.n_groups);
    if (l.n_groups == 1) {
        if (vec) ce_row_stats_kernel<T, true, true><<<grid, kCeThreads, 0, s>>>(z, tgt, tgt_i64, (int)N, V, nc, ng, partial, l.row_stride, ignore_index, lse, loss_rows);
        else ce_row_stats_kernel<T, false, true><<<grid, kCeThreads, 0, s>>>(z, tgt, tgt_i64, (int)N, V, nc, ng, partial, l.row_stride, ignore_index, lse, loss_rows);
        LCE_COUNT_LAUNCH();
        return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
    }
    if (vec) ce_row_stats_kernel<T, true, false><<<grid, kCeThreads, 0, s>>>(z, tgt, tgt_i64, (int)N, V, nc, ng, partial, l.row_stride, ignore_index, lse, loss_rows);
    else ce_row_stats_kernel<T, false, false><<<grid, kCeThreads, 0, s>>>(z, tgt, tgt_i64, (int)N, V, nc, ng, partial, l.row_stride, ignore_index, lse, loss_rows);
    LCE_COUNT_LAUNCH();
    if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    merge_partials_kernel<true><<<static_cast<int>(cdiv(N, kMergeRows)), kMergeRows * kMergeLanes, 0, s>>>(
        partial, ng, l.row_stride, static_cast<int>(N), nullptr, tgt, tgt_i64, ignore_index, lse, loss_rows);
    LCE_COUNT_LAUNCH();
    return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
}

template <class T>
int ce_backward_impl(const void* logits, const void* tgt, int tgt_i64, long long N, long long V, const float* lse,
                     const float* rowscale, void* dlogits, cudaStream_t s) {
    const bool vec = aligned16(logits) && aligned16(dlogits) && (V * sizeof(T)) % 16 == 0;
    const long long n_chunks = cdiv(V, CeTile<T>::kChunk);
    const int grid = static_cast<int>(N * n_chunks);
    if (vec) ce_backward_kernel<T, true><<<grid, kCeThreads, 0, s>>>(static_cast<const T*>(logits), tgt, tgt_i64, V, (int)n_chunks, lse, rowscale, static_cast<T*>(dlogits));
    else ce_backward_kernel<T, false><<<grid, kCeThreads, 0, s>>>(static_cast<const T*>(logits), tgt, tgt_i64, V, (int)n_chunks, lse, rowscale, static_cast<T*>(dlogits));
    LCE_COUNT_LAUNCH();
    return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
}

int check_ce_dims(long long N, long long V, int dtype, int reduction) {
    if (N < 0 || V <= 0) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_F32) return LCE_ERR_ARG;
    if (reduction != LCE_REDUCTION_NONE && reduction != LCE_REDUCTION_MEAN && reduction != LCE_REDUCTION_SUM)
        return LCE_ERR_ARG;
    if (N > 0x7fffff00ll || N * cdiv(V, ce_chunk(dtype)) > 0x7fffff00ll) return LCE_ERR_TOO_LARGE;
    return LCE_OK;
}

}  // namespace
}  // namespace lce

extern "C" {

size_t lce_ce_workspace_bytes(int64_t N, int64_t V, int dtype) {
    if (N < 0 || V <= 0) return 0;
    return ce_layout(N, V, dtype).total;
}

int lce_ce_forward(const void* logits, const void* target, int target_is_i64, int64_t N, int64_t V, int dtype,
                   int64_t ignore_index, int reduction, float* lse, float* loss, float* valid_count, void* ws,
                   size_t ws_bytes, void* stream) {
    int rc = check_ce_dims(N, V, dtype, reduction);
    if (rc) return rc;
    if (N == 0) return LCE_ERR_ARG;  // the empty batch is the caller's business
    if (!logits || !target || !lse || !loss || !ws) return LCE_ERR_ARG;
    DeviceInfo* d;
    if ((rc = device_info(&d))) return rc;
    const CeLayout l = ce_layout(N, V, dtype);
    if (ws_bytes < l.total) return LCE_ERR_WS_TOO_SMALL;
    char* wsc = static_cast<char*>(ws);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* loss_rows = reduction == LCE_REDUCTION_NONE ? loss : reinterpret_cast<float*>(wsc + l.off_loss_rows);
    switch (dtype) {
        case LCE_DTYPE_BF16: rc = ce_forward_impl<__nv_bfloat16>(logits, target, target_is_i64, N, V, ignore_index, l, wsc, lse, loss_rows, s); break;
        case LCE_DTYPE_F16: rc = ce_forward_impl<__half>(logits, target, target_is_i64, N, V, ignore_index, l, wsc, lse, loss_rows, s); break;
        default: rc = ce_forward_impl<float>(logits, target, target_is_i64, N, V, ignore_index, l, wsc, lse, loss_rows, s);
    }
    if (rc) return rc;
    if (reduction != LCE_REDUCTION_NONE || valid_count) {
        reduce_loss_kernel<<<1, 1024, 0, s>>>(loss_rows, target, target_is_i64, static_cast<int>(N), ignore_index,
                                              reduction == LCE_REDUCTION_MEAN ? 1 : 0,
                                              reduction == LCE_REDUCTION_NONE ? nullptr : loss, valid_count);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    return LCE_OK;
}

int lce_ce_backward(const void* logits, const void* target, int target_is_i64, const float* lse,
                    const float* grad_out, int64_t N, int64_t V, int dtype, int64_t ignore_index, int reduction,
                    void* dlogits, void* ws, size_t ws_bytes, void* stream) {
    int rc = check_ce_dims(N, V, dtype, reduction);
    if (rc) return rc;
    if (N == 0) return LCE_OK;
    if (!logits || !target || !lse || !grad_out || !dlogits || !ws) return LCE_ERR_ARG;
    DeviceInfo* d;
    if ((rc = device_info(&d))) return rc;
    const CeLayout l = ce_layout(N, V, dtype);
    if (ws_bytes < l.total) return LCE_ERR_WS_TOO_SMALL;
    char* wsc = static_cast<char*>(ws);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* rowscale = reinterpret_cast<float*>(wsc + l.off_rowscale);
    float* count = reinterpret_cast<float*>(wsc + l.off_count);
    const bool separate_count = reduction == LCE_REDUCTION_MEAN && N > 16384;
    if (separate_count) {
        count_valid_kernel<<<1, 1024, 0, s>>>(target, target_is_i64, static_cast<int>(N), ignore_index, count);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    rowscale_kernel<<<static_cast<int>(cdiv(N, 256)), 256, 0, s>>>(
        target, target_is_i64, static_cast<int>(N), ignore_index, grad_out, reduction == LCE_REDUCTION_NONE ? 1 : 0,
        reduction == LCE_REDUCTION_MEAN ? 1 : 0, separate_count ? count : nullptr, rowscale);
    LCE_COUNT_LAUNCH();
    if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    switch (dtype) {
        case LCE_DTYPE_BF16: return ce_backward_impl<__nv_bfloat16>(logits, target, target_is_i64, N, V, lse, rowscale, dlogits, s);
        case LCE_DTYPE_F16: return ce_backward_impl<__half>(logits, target, target_is_i64, N, V, lse, rowscale, dlogits, s);
        default: return ce_backward_impl<float>(logits, target, target_is_i64, N, V, lse, rowscale, dlogits, s);
    }
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Plain matrix product on the same GEMM cores
// ---------------------------------------------------------------------------------------------
namespace lce {
namespace {

struct MatmulPlan {
    bool use_tc;
    int cg;
    int splits;
    long long slab_floats;
    size_t ws_bytes;
};

MatmulPlan plan_matmul(long long M, long long N, long long K, int dtype, bool aligned, unsigned flags) {
    MatmulPlan p;
    p.cg = cta_group_of(flags);
    p.use_tc = dtype != LCE_DTYPE_F32 && aligned && !(flags & LCE_FLAG_FORCE_SIMT);
    p.splits = p.use_tc ? choose_k_splits(M, N, K, p.cg) : 1;
    p.slab_floats = cdiv(M, 2 * kBM) * 2 * cdiv(N, kBN) * kBM * kBN;
    p.ws_bytes = p.splits > 1 ? static_cast<size_t>(p.splits) * p.slab_floats * sizeof(float) : 0;
    return p;
}

template <class T>
int matmul_impl(const DeviceInfo& d, const MatmulPlan& p, const Mat& a, bool a_mn, const Mat& b, bool b_mn, void* c,
                long long M, long long N, long long K, long long ldc, void* ws, cudaStream_t s) {
    typename EpiStore<T>::Params ep;
    ep.out = static_cast<T*>(c);
    ep.ldo = ldc;
    ep.rows = static_cast<int>(M);
    ep.cols = static_cast<int>(N);
    ep.scratch = static_cast<float*>(ws);
    ep.mode = p.splits > 1 ? kStoreSlice : kStoreDirect;
    ep.slab_floats = p.slab_floats;
    ep.peer_world = 0;
    ep.wide = wide_stores(c, ldc);
    if (!p.use_tc) return launch_simt<T, EpiStore<T>>(d, a, a_mn, b, b_mn, M, N, K, ep, s);
    int rc = LCE_ERR_ARG;
    if constexpr (sizeof(T) == 2) {
        constexpr bool kBf16 = std::is_same<T, __nv_bfloat16>::value;
        // tiles that run together share a B panel when there are many row tiles, an A panel otherwise
        const int m_fastest = cdiv(M, kBM) >= cdiv(N, kBN) ? 1 : 0;
        if (!a_mn && !b_mn) rc = launch_tc<false, false, kBf16, EpiStore<T>>(d, p.cg, a, b, M, N, K, m_fastest, ep, s, p.splits);
        else if (!a_mn && b_mn) rc = launch_tc<false, true, kBf16, EpiStore<T>>(d, p.cg, a, b, M, N, K, m_fastest, ep, s, p.splits);
        else if (a_mn && !b_mn) rc = launch_tc<true, false, kBf16, EpiStore<T>>(d, p.cg, a, b, M, N, K, m_fastest, ep, s, p.splits);
        else rc = launch_tc<true, true, kBf16, EpiStore<T>>(d, p.cg, a, b, M, N, K, m_fastest, ep, s, p.splits);
        if (rc == LCE_OK && p.splits > 1) {
            const int m_tiles = static_cast<int>(cdiv(M, kBM)), n_tiles = static_cast<int>(cdiv(N, kBN));
            const long long quads = static_cast<long long>(m_tiles) * n_tiles * (kBN / 4) * kBM;
            const int blocks = static_cast<int>(cdiv(quads, 256) < 4096 ? cdiv(quads, 256) : 4096);
            const cudaError_t err = launch_dependent(
                splitk_reduce_kernel<T>, blocks, 256, s, static_cast<const float*>(ep.scratch), p.splits, p.slab_floats,
                m_tiles, n_tiles, static_cast<int>(kBN), static_cast<int>(M), static_cast<int>(N), ep.out, ldc);
            LCE_COUNT_LAUNCH();
            if (cuda_failed(err)) rc = LCE_ERR_CUDA;
        }
    }
    return rc;
}

bool matmul_aligned(const void* a, const void* b, long long lda, long long ldb) {
    return aligned16(a) && aligned16(b) && lda % 8 == 0 && ldb % 8 == 0;
}

}  // namespace
}  // namespace lce

extern "C" {

size_t lce_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype, unsigned flags) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return plan_matmul(M, N, K, dtype, true, flags).ws_bytes;
}

int lce_matmul(const void* a, const void* b, void* c, int64_t M, int64_t N, int64_t K, int a_mn_major, int64_t lda,
               int b_mn_major, int64_t ldb, int64_t ldc, int dtype, void* ws, size_t ws_bytes, unsigned flags,
               void* stream) {
    if (M < 0 || N < 0 || K < 0 || lda <= 0 || ldb <= 0 || ldc <= 0) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_F32) return LCE_ERR_ARG;
    if (M > 0x7fffff00ll || N > 0x7fffff00ll || K > 0x7fffff00ll) return LCE_ERR_TOO_LARGE;
    if (M == 0 || N == 0) return LCE_OK;
    if (!c) return LCE_ERR_ARG;
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 0) {  // an empty contraction is all zeros
        if (ldc != N) return LCE_ERR_ARG;
        return cudaMemsetAsync(c, 0, static_cast<size_t>(M) * N * elem_size(dtype), s) == cudaSuccess ? LCE_OK : LCE_ERR_CUDA;
    }
    if (!a || !b) return LCE_ERR_ARG;
    const bool aligned = matmul_aligned(a, b, lda, ldb);
    if ((flags & LCE_FLAG_FORCE_TC) && (dtype == LCE_DTYPE_F32 || !aligned)) return dtype == LCE_DTYPE_F32 ? LCE_ERR_ARG : LCE_ERR_ALIGN;
    const MatmulPlan p = plan_matmul(M, N, K, dtype, aligned, flags);
    if (p.ws_bytes > 0 && (!ws || ws_bytes < p.ws_bytes)) return LCE_ERR_WS_TOO_SMALL;
    const Mat am = a_mn_major ? Mat{a, K, M, lda} : Mat{a, M, K, lda};
    const Mat bm = b_mn_major ? Mat{b, K, N, ldb} : Mat{b, N, K, ldb};
    switch (dtype) {
        case LCE_DTYPE_BF16: return matmul_impl<__nv_bfloat16>(*d, p, am, a_mn_major, bm, b_mn_major, c, M, N, K, ldc, ws, s);
        case LCE_DTYPE_F16: return matmul_impl<__half>(*d, p, am, a_mn_major, bm, b_mn_major, c, M, N, K, ldc, ws, s);
        default: return matmul_impl<float>(*d, p, am, a_mn_major, bm, b_mn_major, c, M, N, K, ldc, ws, s);
    }
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Consumers of dW: AdamW step and the sum of squares for gradient clipping
// ---------------------------------------------------------------------------------------------
extern "C" {

int lce_adamw_step(void* param, const void* grad, float* exp_avg, float* exp_avg_sq, int64_t n, int dtype, float lr,
                   float beta1, float beta2, float eps, float weight_decay, int64_t step, const float* grad_scale,
                   void* stream) {
    if (n < 0 || step < 1) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_F32) return LCE_ERR_ARG;
    if (n == 0) return LCE_OK;
    if (!param || !grad || !exp_avg || !exp_avg_sq) return LCE_ERR_ARG;
    if (!aligned16(param) || !aligned16(grad) || !aligned16(exp_avg) || !aligned16(exp_avg_sq)) return LCE_ERR_ALIGN;
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    // bias corrections in double, as Python computes them for the reference kernel
    const float bc1 = static_cast<float>(1.0 - pow(static_cast<double>(beta1), static_cast<double>(step)));
    const float bc2 = static_cast<float>(1.0 - pow(static_cast<double>(beta2), static_cast<double>(step)));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long vecs = n / (16 / static_cast<long long>(elem_size(dtype))) + 1;
    const long long want = cdiv(vecs, kOptThreads);  // one 16-byte vector per thread: nothing but loads in flight
    const int blocks = static_cast<int>(want < 0x7fffffffll ? want : 0x7fffffffll);
    switch (dtype) {
        case LCE_DTYPE_BF16:
            adamw_step_kernel<__nv_bfloat16><<<blocks, kOptThreads, 0, s>>>(static_cast<__nv_bfloat16*>(param), static_cast<const __nv_bfloat16*>(grad), exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
            break;
        case LCE_DTYPE_F16:
            adamw_step_kernel<__half><<<blocks, kOptThreads, 0, s>>>(static_cast<__half*>(param), static_cast<const __half*>(grad), exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
            break;
        default:
            adamw_step_kernel<float><<<blocks, kOptThreads, 0, s>>>(static_cast<float*>(param), static_cast<const float*>(grad), exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
    }
    LCE_COUNT_LAUNCH();
    return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
}

size_t lce_sumsq_workspace_bytes(void) { return kSumsqBlocks * sizeof(float); }

int lce_sumsq(const void* x, int64_t n, int dtype, float* out, int accumulate, void* ws, size_t ws_bytes, void* stream) {
    if (n < 0 || !out) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_F32) return LCE_ERR_ARG;
    if (!ws || ws_bytes < kSumsqBlocks * sizeof(float)) return LCE_ERR_WS_TOO_SMALL;
    if (n > 0 && (!x || !aligned16(x))) return x ? LCE_ERR_ALIGN : LCE_ERR_ARG;
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* partials = static_cast<float*>(ws);
    switch (dtype) {
        case LCE_DTYPE_BF16: sumsq_partial_kernel<__nv_bfloat16><<<kSumsqBlocks, kOptThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, partials); break;
        case LCE_DTYPE_F16: sumsq_partial_kernel<__half><<<kSumsqBlocks, kOptThreads, 0, s>>>(static_cast<const __half*>(x), n, partials); break;
        default: sumsq_partial_kernel<float><<<kSumsqBlocks, kOptThreads, 0, s>>>(static_cast<const float*>(x), n, partials);
    }
    LCE_COUNT_LAUNCH();
    if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    sumsq_final_kernel<<<1, 1024, 0, s>>>(partials, kSumsqBlocks, out, accumulate);
    LCE_COUNT_LAUNCH();
    return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// RMSNorm / residual RMSNorm
// ---------------------------------------------------------------------------------------------
namespace lce {
namespace {

struct RmsShape {
    bool wide;    // row does not fit the register-resident kernels
    bool vector;  // 16-byte accesses are legal
    int vpt, threads;
    int rows;     // rows one CTA handles per step (RmsRows<vpt>)
};

RmsShape rms_shape(long long H, int dtype, bool all_aligned, int n_streams = 1) {
    const long long vec = 16 / static_cast<long long>(elem_size(dtype));
    const int max_vpt = RmsTile<float>::kMaxVpt;
    RmsShape r;
    r.vector = all_aligned && (H % vec) == 0;
    const long long nvec = cdiv(H, vec);
    r.wide = nvec > static_cast<long long>(max_vpt) * kRmsMaxThreads;
    r.vpt = 1;
    static const int kThreadTarget = [] {  // HELION_B200_RMS_THREADS: threads per row aimed for (tuning knob)
        const char* e = getenv("HELION_B200_RMS_THREADS");
        return e && atoi(e) >= 32 && atoi(e) <= kRmsMaxThreads ? atoi(e) : kRmsMaxThreads;
    }();
    while (r.vpt < max_vpt && cdiv(nvec, r.vpt) > kThreadTarget) r.vpt *= 2;
    // with two or three tensors streaming in, rows of 129..256 vectors measured 2-5 % faster on 128 threads
    // with two vectors each than on 256 threads with one
    if (n_streams >= 2 && r.vpt == 1 && nvec > 128) r.vpt = 2;
    const long long threads = cdiv(cdiv(nvec, r.vpt), 32) * 32;
    r.threads = r.wide ? kRmsMaxThreads : static_cast<int>(threads < 32 ? 32 : threads);
    r.rows = r.wide ? 1 : (r.vpt >= 4 ? 1 : 4 / r.vpt);
    return r;
}

// CTAs for a row kernel of `threads` threads: enough to keep every SM's thread slots full.
int rms_grid(const DeviceInfo& d, long long n_rows, int threads, long long cap) {
    // HELION_B200_RMS_GRID_MULT (tuning knob): grid = this many times the resident CTAs; 0 = one CTA per row
    // group, i.e. no persistence at all (the hardware deals the CTAs to the SMs as they retire)
    static const int kGridMult = [] { const char* e = getenv("HELION_B200_RMS_GRID_MULT"); return e ? atoi(e) : 4; }();
    long long per_sm = 2048 / threads;
    if (per_sm > 16) per_sm = 16;
    long long g = static_cast<long long>(d.sm_count) * per_sm;
    g = kGridMult > 0 ? g * kGridMult : n_rows;
    if (cap > 0 && g > cap) g = cap;
    return static_cast<int>(n_rows < g ? n_rows : g);
}

// Shared-memory ring of a ring kernel: CTAs per SM by thread count, the per-CTA share of the SM's
// shared memory, and as many stages (2..4) as fit.
constexpr long long kRmsRingMinBytes = 16ll << 20;  // forward only; the backward ring wins at every size measured
constexpr long long kRmsRingMinRowBytes = 8192;

struct RmsRingPlan {
    int ctas_per_sm, stages;
    int rows;  // rows per stage (RmsRingRows<vpt, n_streams>)
    size_t smem;
};

RmsRingPlan rms_ring_plan(const RmsShape& sh, long long H, int dtype, int n_streams, bool forward) {
    RmsRingPlan p;
    // tuning knobs: HELION_B200_RMS_CTAS = CTAs per SM, HELION_B200_RMS_STAGES = most stages per ring
    static const int kCtasOverride = [] { const char* e = getenv("HELION_B200_RMS_CTAS"); return e ? atoi(e) : 0; }();
    static const int kStagesCap = [] {
        const char* e = getenv("HELION_B200_RMS_STAGES");
        return e && atoi(e) >= 2 && atoi(e) <= kRmsMaxStages ? atoi(e) : kRmsMaxStages;
    }();
    // threads per SM the registers allow: the forward kernels stay under 85 registers, the backward ones under 128
    p.ctas_per_sm = kCtasOverride > 0 ? kCtasOverride : (forward ? 768 : 512) / sh.threads;
    if (p.ctas_per_sm < 2) p.ctas_per_sm = 2;
    if (p.ctas_per_sm > 8) p.ctas_per_sm = 8;
    const int target = n_streams == 1 ? 8 : 4;
    p.rows = sh.vpt >= target ? 1 : target / sh.vpt;
    const size_t stage = static_cast<size_t>(p.rows) * n_streams * H * elem_size(dtype);
    for (;; --p.ctas_per_sm) {  // fewer, larger rings until two stages fit
        const size_t budget = kRmsRingBytesPerSm / p.ctas_per_sm - 2048;  // static shared memory and slack
        const long long st = static_cast<long long>(budget / stage);
        p.stages = static_cast<int>(st > kStagesCap ? kStagesCap : st);
        if (p.stages >= 2 || p.ctas_per_sm == 2) break;
    }
    p.smem = p.stages * stage;
    return p;
}

// Opt a kernel into more than 48 KB of dynamic shared memory, once per device and kernel.
template <auto Kernel>
int rms_ring_opt_in(const DeviceInfo& d) {
    static std::atomic<bool> done[kMaxDevices];
    if (!done[d.index].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRmsRingBytesPerSm / 2) !=
            cudaSuccess)
            return LCE_ERR_CUDA;
        done[d.index].store(true, std::memory_order_release);
    }
    return LCE_OK;
}

int rms_ring_grid(const DeviceInfo& d, const RmsShape& sh, const RmsRingPlan& rp, long long n_rows, long long cap) {
    long long g = static_cast<long long>(d.sm_count) * rp.ctas_per_sm;
    if (cap > 0 && g > cap) g = cap;
    const long long groups = cdiv(n_rows, rp.rows);
    return static_cast<int>(groups < g ? groups : g);
}

// Which form a forward / backward takes (the launch code and lce_rmsnorm_plan both ask here).
// Forward: plain rmsnorm of rows of 8 KB and more streams through the shared-memory ring once the input
// reaches kRmsRingMinBytes; narrower rows, small inputs and the residual form are faster on the register
// kernels (measured: the ring's set-up costs ~2 us, and with two tensors streaming in it gains nothing).
bool rms_forward_uses_ring(const RmsShape& sh, long long n_rows, long long H, int dtype, bool residual, RmsRingPlan* rp) {
    static const long long kRingMinBytes = [] {  // HELION_B200_RMS_RING_MIN_MB overrides (tuning knob)
        const char* e = getenv("HELION_B200_RMS_RING_MIN_MB");
        return e ? atoll(e) << 20 : kRmsRingMinBytes;
    }();
    const long long row_bytes = H * static_cast<long long>(elem_size(dtype));
    if (residual || !sh.vector || sh.wide || row_bytes < kRmsRingMinRowBytes || n_rows * row_bytes < kRingMinBytes)
        return false;
    *rp = rms_ring_plan(sh, H, dtype, 1, true);
    return rp->stages >= 2;
}

// Backward: the ring whenever 16-byte copies are legal and two stages fit.
bool rms_backward_uses_ring(const RmsShape& sh, long long H, int dtype, bool has_dres, RmsRingPlan* rp) {
    if (!sh.vector || sh.wide) return false;
    *rp = rms_ring_plan(sh, H, dtype, has_dres ? 3 : 2, false);
    return rp->stages >= 2;
}

template <class T, bool RESIDUAL>
int rms_forward_launch(const DeviceInfo& d, const RmsShape& sh, const void* x, const void* residual,
                       const void* weight, void* out, void* residual_out, float* rstd, long long n_rows,
                       long long H, float eps, cudaStream_t s) {
    const T* xp = static_cast<const T*>(x);
    const T* rp = static_cast<const T*>(residual);
    const T* wp = static_cast<const T*>(weight);
    T* op = static_cast<T*>(out);
    T* rop = static_cast<T*>(residual_out);
    const int n = static_cast<int>(n_rows), h = static_cast<int>(H);
    if constexpr (!RESIDUAL) {
        // Plain forward of 16-byte-aligned rows of 8 KB and more: one small CTA per row (rms_forward_row_kernel);
        // narrower rows measured faster on the register kernels below, which pack several rows into a CTA.
        // HELION_B200_RMS_ROW=0 (tuning knob) falls back to the ring / register kernels for every width.
        static const int kRowKernel = [] { const char* e = getenv("HELION_B200_RMS_ROW"); return e ? atoi(e) : 1; }();
        constexpr long long kVec = 16 / sizeof(T);
        const long long nvec = H / kVec;
        if (kRowKernel != 0 && sh.vector && !sh.wide && H * static_cast<long long>(sizeof(T)) >= 8192 && nvec <= 256 * 8) {
            const int threads = nvec <= 128 * 4 ? 128 : 256;
            const long long per_thread = cdiv(nvec, threads);
            const int grid = static_cast<int>(n_rows);
#define LCE_RMS_ROW(VPT, THREADS) \
    rms_forward_row_kernel<T, VPT, THREADS><<<grid, THREADS, 0, s>>>(xp, wp, op, rstd, n, h, eps)
            if (threads == 128) {  // 8 KB rows: exactly four vectors per thread
                LCE_RMS_ROW(4, 128);
            } else {
                if (per_thread <= 4) LCE_RMS_ROW(4, 256);
                else LCE_RMS_ROW(8, 256);
            }
#undef LCE_RMS_ROW
            LCE_COUNT_LAUNCH();
            return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
        }
    }
    {
        RmsRingPlan rp;
        if (rms_forward_uses_ring(sh, n_rows, H, sizeof(T) == 4 ? LCE_DTYPE_F32 : LCE_DTYPE_F16, RESIDUAL, &rp)) {
            static std::atomic<bool> hint_set[kMaxDevices];
            if (!hint_set[d.index].load(std::memory_order_acquire)) {
                const char* e = getenv("HELION_B200_RMS_HINT");
                const int hint = e ? atoi(e) : 0;
                if (hint != 0 && cudaMemcpyToSymbol(g_rms_hint, &hint, sizeof(int)) != cudaSuccess) return LCE_ERR_CUDA;
                hint_set[d.index].store(true, std::memory_order_release);
            }
            const int grid = rms_ring_grid(d, sh, rp, n_rows, 0);
            int rc = LCE_OK;
#define LCE_RMS_RING_FWD(VPT)                                                                             \
    rc = rms_ring_opt_in<rms_ring_forward_kernel<T, VPT>>(d);                                             \
    if (rc == LCE_OK)                                                                                      \
        rms_ring_forward_kernel<T, VPT><<<grid, sh.threads, rp.smem, s>>>(xp, wp, op, rstd, n, h, eps, rp.stages, \
                                                                          d.status_ptr)
            switch (sh.vpt) {  // rows of 8 KB and more never have one vector per thread
                case 2: LCE_RMS_RING_FWD(2); break;
                case 4: LCE_RMS_RING_FWD(4); break;
                case 8: LCE_RMS_RING_FWD(8); break;
                default: return LCE_ERR_ARG;
            }
#undef LCE_RMS_RING_FWD
            if (rc != LCE_OK) return rc;
            LCE_COUNT_LAUNCH();
            return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
        }
    }
    const int grid = rms_grid(d, cdiv(n_rows, sh.rows), sh.threads, 0);
#define LCE_RMS_FWD(VPT, VECTOR) \
    rms_forward_kernel<T, VPT, VECTOR, RESIDUAL><<<grid, sh.threads, 0, s>>>(xp, rp, wp, op, rop, rstd, n, h, eps)
    if (sh.wide) {
        rms_forward_wide_kernel<T, RESIDUAL><<<grid, sh.threads, 0, s>>>(xp, rp, wp, op, rop, rstd, n, h, eps);
    } else if (sh.vector) {
        switch (sh.vpt) {
            case 1: LCE_RMS_FWD(1, true); break;
            case 2: LCE_RMS_FWD(2, true); break;
            case 4: LCE_RMS_FWD(4, true); break;
            default: LCE_RMS_FWD(8, true);
        }
    } else {
        switch (sh.vpt) {
            case 1: LCE_RMS_FWD(1, false); break;
            case 2: LCE_RMS_FWD(2, false); break;
            case 4: LCE_RMS_FWD(4, false); break;
            default: LCE_RMS_FWD(8, false);
        }
    }
#undef LCE_RMS_FWD
    LCE_COUNT_LAUNCH();
    return (cuda_failed(cudaGetLastError()) ? LCE_ERR_CUDA : LCE_OK);
}

// Rows of partial dweight sums the backward writes for (n_rows, H): one per CTA of the row kernel.
long long rms_partial_rows(long long n_rows, long long H, int dtype) {
    const RmsShape sh = rms_shape(H, dtype, true);
    if (sh.wide) {
        const long long blocks = cdiv(n_rows, 128);
        return blocks < kRmsMaxPartials ? blocks : kRmsMaxPartials;
    }
    return n_rows < kRmsMaxPartials ? n_rows : kRmsMaxPartials;
}

template <class T>
int rms_backward_launch(const DeviceInfo& d, const RmsShape& sh, const void* dy, const void* x, const void* weight,
                        const float* rstd, const void* dres, void* dx, void* dweight, long long n_rows,
                        long long H, float eps, float* partial, float* rstd_ws, cudaStream_t s) {
    const T* dyp = static_cast<const T*>(dy);
    const T* xp = static_cast<const T*>(x);
    const T* wp = static_cast<const T*>(weight);
    const T* drp = static_cast<const T*>(dres);
    T* dxp = static_cast<T*>(dx);
    const int n = static_cast<int>(n_rows), h = static_cast<int>(H);
    float* part = dweight != nullptr ? partial : nullptr;
    int n_partials = 0;
    if (sh.wide) {
        const int grid = rms_grid(d, n_rows, sh.threads, 0);
        float* rs = dweight != nullptr ? rstd_ws : nullptr;
        rms_backward_wide_kernel<T><<<grid, sh.threads, 0, s>>>(dyp, xp, wp, rstd, drp, dxp, rs, n, h, eps);
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
        if (dweight != nullptr) {
            n_partials = static_cast<int>(rms_partial_rows(n_rows, H, sizeof(T) == 4 ? LCE_DTYPE_F32 : LCE_DTYPE_F16));
            const int rows_per_block = static_cast<int>(cdiv(n_rows, n_partials));
            n_partials = static_cast<int>(cdiv(n_rows, rows_per_block));
            dim3 g(static_cast<unsigned>(cdiv(H, 256)), static_cast<unsigned>(n_partials));
            rms_dw_wide_kernel<T><<<g, 256, 0, s>>>(dyp, xp, rs, part, n, h, rows_per_block);
            LCE_COUNT_LAUNCH();
            if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
        }
    } else if (RmsRingPlan rp; rms_backward_uses_ring(sh, H, sizeof(T) == 4 ? LCE_DTYPE_F32 : LCE_DTYPE_F16, drp != nullptr, &rp)) {
        const int grid = rms_ring_grid(d, sh, rp, n_rows, kRmsMaxPartials);
        n_partials = grid;
        int rc = LCE_OK;
#define LCE_RMS_RING_BWD(VPT, DRES)                                                                              \
    rc = rms_ring_opt_in<rms_ring_backward_kernel<T, VPT, DRES>>(d);                                             \
    if (rc == LCE_OK)                                                                                             \
        rms_ring_backward_kernel<T, VPT, DRES><<<grid, sh.threads, rp.smem, s>>>(dyp, xp, wp, rstd, drp, dxp, part, n, \
                                                                                 h, eps, rp.stages, d.status_ptr)
        if (drp != nullptr) {
            switch (sh.vpt) {
                case 1: LCE_RMS_RING_BWD(1, true); break;
                case 2: LCE_RMS_RING_BWD(2, true); break;
                case 4: LCE_RMS_RING_BWD(4, true); break;
                default: LCE_RMS_RING_BWD(8, true);
            }
        } else {
            switch (sh.vpt) {
                case 1: LCE_RMS_RING_BWD(1, false); break;
                case 2: LCE_RMS_RING_BWD(2, false); break;
                case 4: LCE_RMS_RING_BWD(4, false); break;
                default: LCE_RMS_RING_BWD(8, false);
            }
        }
#undef LCE_RMS_RING_BWD
        if (rc != LCE_OK) return rc;
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    } else {
        const int grid = rms_grid(d, cdiv(n_rows, sh.rows), sh.threads, kRmsMaxPartials);
        n_partials = grid;
#define LCE_RMS_BWD(VPT, VECTOR) \
    rms_backward_kernel<T, VPT, VECTOR><<<grid, sh.threads, 0, s>>>(dyp, xp, wp, rstd, drp, dxp, part, n, h, eps)
        if (sh.vector) {
            switch (sh.vpt) {
                case 1: LCE_RMS_BWD(1, true); break;
                case 2: LCE_RMS_BWD(2, true); break;
                case 4: LCE_RMS_BWD(4, true); break;
                default: LCE_RMS_BWD(8, true);
            }
        } else {
            switch (sh.vpt) {
                case 1: LCE_RMS_BWD(1, false); break;
                case 2: LCE_RMS_BWD(2, false); break;
                case 4: LCE_RMS_BWD(4, false); break;
                default: LCE_RMS_BWD(8, false);
            }
        }
#undef LCE_RMS_BWD
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    if (dweight != nullptr) {
        dim3 block(32, 8);
        rms_dw_reduce_kernel<T><<<static_cast<unsigned>(cdiv(H, 32)), block, 0, s>>>(part, n_partials, h,
                                                                                     static_cast<T*>(dweight));
        LCE_COUNT_LAUNCH();
        if (cuda_failed(cudaGetLastError())) return LCE_ERR_CUDA;
    }
    return LCE_OK;
}

inline size_t rms_partial_bytes(long long n_rows, long long H, int dtype) {
    return (static_cast<size_t>(rms_partial_rows(n_rows, H, dtype)) * static_cast<size_t>(H) * sizeof(float) + 255) /
           256 * 256;
}

}  // namespace
}  // namespace lce

extern "C" {

int lce_rmsnorm_forward(const void* x, const void* residual, const void* weight, void* out, void* residual_out,
                        float* rstd, int64_t n_rows, int64_t hidden, float eps, int dtype, void* stream) {
    using namespace lce;
    // row indices are ints in the kernels, and a CTA steps past the end by up to grid x rows-per-step before it stops
    if (n_rows < 0 || hidden < 1 || n_rows > 0x7fff0000ll || hidden > 0x7fffffffll / 16) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_F32) return LCE_ERR_ARG;
    if ((residual == nullptr) != (residual_out == nullptr)) return LCE_ERR_ARG;
    if (n_rows == 0) return LCE_OK;
    if (!x || !weight || !out) return LCE_ERR_ARG;
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    const bool al = aligned16(x) && aligned16(weight) && aligned16(out) &&
                    (!residual || (aligned16(residual) && aligned16(residual_out)));
    const RmsShape sh = rms_shape(hidden, dtype, al, residual ? 2 : 1);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define LCE_RMS_GO(T)                                                                                              \
    (residual ? rms_forward_launch<T, true>(*d, sh, x, residual, weight, out, residual_out, rstd, n_rows, hidden, \
                                            eps, s)                                                                \
              : rms_forward_launch<T, false>(*d, sh, x, nullptr, weight, out, nullptr, rstd, n_rows, hidden, eps, s))
    switch (dtype) {
        case LCE_DTYPE_BF16: return LCE_RMS_GO(__nv_bfloat16);
        case LCE_DTYPE_F16: return LCE_RMS_GO(__half);
        default: return LCE_RMS_GO(float);
    }
#undef LCE_RMS_GO
}

int lce_rmsnorm_plan(int64_t n_rows, int64_t hidden, int dtype, int op, int aligned, int sm_count, int64_t* out) {
    using namespace lce;
    if (!out || n_rows < 1 || hidden < 1 || hidden > 0x7fffffffll / 16 || op < 0 || op > 3 || sm_count < 1) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_F32) return LCE_ERR_ARG;
    const bool forward = op < 2;
    const int n_streams = op == 0 ? 1 : op == 1 ? 2 : op;
    const RmsShape sh = rms_shape(hidden, dtype, aligned != 0, n_streams);
    DeviceInfo d;
    d.sm_count = sm_count;
    RmsRingPlan rp{};
    const bool ring = forward ? rms_forward_uses_ring(sh, n_rows, hidden, dtype, op == 1, &rp)
                              : rms_backward_uses_ring(sh, hidden, dtype, op == 3, &rp);
    out[0] = ring ? 0 : sh.wide ? 2 : 1;
    out[1] = sh.vpt;
    out[2] = sh.threads;
    out[3] = ring ? rp.rows : sh.rows;
    out[4] = ring ? rp.ctas_per_sm : 0;
    out[5] = ring ? rp.stages : 0;
    out[6] = ring ? static_cast<int64_t>(rp.smem) : 0;
    const long long cap = forward ? 0 : kRmsMaxPartials;
    out[7] = ring ? rms_ring_grid(d, sh, rp, n_rows, cap)
                  : rms_grid(d, sh.wide ? n_rows : cdiv(n_rows, sh.rows), sh.threads, sh.wide && !forward ? 0 : cap);
    return LCE_OK;
}

size_t lce_rmsnorm_backward_workspace_bytes(int64_t n_rows, int64_t hidden, int dtype) {
    using namespace lce;
    if (n_rows <= 0 || hidden < 1) return 0;
    return rms_partial_bytes(n_rows, hidden, dtype) + (static_cast<size_t>(n_rows) * sizeof(float) + 255) / 256 * 256;
}

int lce_rmsnorm_backward(const void* dy, const void* x, const void* weight, const float* rstd, const void* dresidual,
                         void* dx, void* dweight, int64_t n_rows, int64_t hidden, float eps, int dtype, void* ws,
                         size_t ws_bytes, void* stream) {
    using namespace lce;
    // row indices are ints in the kernels, and a CTA steps past the end by up to grid x rows-per-step before it stops
    if (n_rows < 0 || hidden < 1 || n_rows > 0x7fff0000ll || hidden > 0x7fffffffll / 16) return LCE_ERR_ARG;
    if (dtype != LCE_DTYPE_BF16 && dtype != LCE_DTYPE_F16 && dtype != LCE_DTYPE_F32) return LCE_ERR_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n_rows == 0) {  // dweight of an empty batch is zero
        if (dweight && cudaMemsetAsync(dweight, 0, static_cast<size_t>(hidden) * elem_size(dtype), s) != cudaSuccess)
            return LCE_ERR_CUDA;
        return LCE_OK;
    }
    if (!dy || !x || !weight || !dx) return LCE_ERR_ARG;
    float* partial = nullptr;
    float* rstd_ws = nullptr;
    if (dweight != nullptr) {
        if (!ws || ws_bytes < lce_rmsnorm_backward_workspace_bytes(n_rows, hidden, dtype)) return LCE_ERR_WS_TOO_SMALL;
        if (!aligned16(ws)) return LCE_ERR_ALIGN;
        partial = static_cast<float*>(ws);
        rstd_ws = reinterpret_cast<float*>(static_cast<char*>(ws) + rms_partial_bytes(n_rows, hidden, dtype));
    }
    DeviceInfo* d;
    int rc = device_info(&d);
    if (rc) return rc;
    const bool al = aligned16(dy) && aligned16(x) && aligned16(weight) && aligned16(dx) &&
                    (!dresidual || aligned16(dresidual));
    const RmsShape sh = rms_shape(hidden, dtype, al, dresidual ? 3 : 2);
    switch (dtype) {
        case LCE_DTYPE_BF16:
            return rms_backward_launch<__nv_bfloat16>(*d, sh, dy, x, weight, rstd, dresidual, dx, dweight, n_rows, hidden,
                                                      eps, partial, rstd_ws, s);
        case LCE_DTYPE_F16:
            return rms_backward_launch<__half>(*d, sh, dy, x, weight, rstd, dresidual, dx, dweight, n_rows, hidden, eps,
                                               partial, rstd_ws, s);
        default:
            return rms_backward_launch<float>(*d, sh, dy, x, weight, rstd, dresidual, dx, dweight, n_rows, hidden, eps,
                                              partial, rstd_ws, s);
    }
}

}  // extern "C"
