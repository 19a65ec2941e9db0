// Host side of the C ABI: argument checks, knob -> kernel variant, TMA descriptors, launch.
//
// Takes the place of the reference's launcher and its 160-way template dispatch
// (csrc/kernels/fused_moe_w8a8/fused_moe_w8a8_up_down_acc.cu:1100-1303).  Differences that matter
// to a caller: tensor maps are encoded once per (pointer, shape) and cached instead of per call
// (:1135-1178), every CUDA / driver return code is checked and reported instead of exit()
// (:14-21, :1143, :1167), and block_m only selects among four padded tile variants.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "../../include/alpha_moe_b200.h"
#include "capi_internal.h"
#include "fused_moe_kernel.cuh"
#include "fused_moe_kernel_tm.cuh"

namespace {

thread_local std::string g_last_error;

}  // namespace

namespace amoe_capi {
int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}
}  // namespace amoe_capi

namespace {
using amoe_capi::fail;

#define CUDA_TRY(expr)                                                                             \
    do {                                                                                           \
        cudaError_t err__ = (expr);                                                                \
        if (err__ != cudaSuccess)                                                                  \
            return fail(ALPHA_MOE_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));      \
    } while (0)

__device__ amoe::KernelStatus g_status;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn* out) {
    static EncodeTiledFn fn = nullptr;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres));
        if (qres != cudaDriverEntryPointSuccess || !p)
            return fail(ALPHA_MOE_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    *out = fn;
    return ALPHA_MOE_OK;
}

struct MapSet {
    CUtensorMap w, w2;      // boxes of 256 rows of w and of 128 rows of w2, each 128 bytes wide
};
using MapKey = std::tuple<int, const void*, const void*, int, int, int>;  // device, w, w2, E, N, K

int encode_map(EncodeTiledFn enc, CUtensorMap* m, const void* base, cuuint64_t inner, cuuint64_t rows, cuuint64_t experts,
               cuuint32_t box_rows, const char* what) {
    cuuint64_t dims[3] = {inner, rows, experts};
    cuuint64_t strides[2] = {inner, rows * inner};
    cuuint32_t box[3] = {128, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ALPHA_MOE_E_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
    return ALPHA_MOE_OK;
}

// Tensor maps depend only on the weight pointers and shapes, so a serving process encodes them once per
// layer.  The cache is bounded (cleared on overflow); the maps are handed out by value, under the lock, so
// that no caller ever holds a pointer into it.
int get_maps(int device, const void* w, const void* w2, int E, int N, int K, MapSet* out) {
    static std::map<MapKey, MapSet> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    MapKey key{device, w, w2, E, N, K};
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return ALPHA_MOE_OK;
    }
    EncodeTiledFn enc;
    if (int rc = get_encode_fn(&enc)) return rc;
    MapSet ms;
    const cuuint64_t I = static_cast<cuuint64_t>(N) / 2, Kk = K, Nn = N, Ee = E;
    // w [E][N][K]: box = consecutive (interleaved) rows x 128 bytes of K
    if (int rc = encode_map(enc, &ms.w, w, Kk, Nn, Ee, 256, "w")) return rc;
    // w2 [E][K][I]: box = hidden rows x 128 bytes of one intermediate slice; rows past K read zero
    if (int rc = encode_map(enc, &ms.w2, w2, I, Kk, Ee, 128, "w2")) return rc;
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, ms);
    *out = ms;
    return ALPHA_MOE_OK;
}

constexpr int kMaxKsplit = 8;        // portable cluster size limit

// Facts about a device that never change, looked up once: the SM count, the address of the status word and how many
// clusters of 2..8 CTAs of the small-batch kernel the device can hold at the same time - with one CTA per SM (deep
// ring) and with two (a ring shallow enough for two CTAs to share an SM's shared memory).
struct ClusterCapacity {
    int one_per_sm[kMaxKsplit + 1] = {};
    int two_per_sm[kMaxKsplit + 1] = {};
};
struct DeviceFacts {
    int sms = 0;
    amoe::KernelStatus* status = nullptr;
    ClusterCapacity clusters;
};
constexpr int kMaxDevices = 64;

constexpr int kMaxDynSmem = 232448;  // 227 KB opt-in limit per CTA on sm_100
constexpr int kPairDynSmem = 115712;  // what each of two co-resident CTAs may use (228 KB per SM, 1 KB reserved per CTA)

int padded_block_m(int block_m) { return block_m <= 16 ? 16 : block_m <= 32 ? 32 : block_m <= 64 ? 64 : 128; }

// Blocks of more than 64 assignments run the token-major kernel (tokens on the TMEM lanes).
bool token_major(int block_m) { return block_m > 64; }

// Ring depth = the `stages` knob, lowered until the plan fits in shared memory.
int plan(int K, int block_m, int stages, int spc, int ksplit, int* depth, int* bmp, int* smem_bytes) {
    const int kc = K / 128;
    const int b = padded_block_m(block_m);
    int s = stages;
    for (; s >= 1; --s) {
        const int need = static_cast<int>(token_major(block_m) ? amoe::smem_plan_tm(s, kc, spc).total
                                                               : amoe::smem_plan(b, s, kc, spc, ksplit).total);
        if (need <= kMaxDynSmem) {
            *depth = s;
            *bmp = b;
            *smem_bytes = need;
            return ALPHA_MOE_OK;
        }
    }
    return fail(ALPHA_MOE_E_ARG, "K=%d block_m=%d does not fit in shared memory even with one stage", K, block_m);
}

// Opts a kernel into the large dynamic shared-memory window once per device (atomically: several host threads
// may launch at the same time).
template <typename Kern>
int ensure_smem_attr(Kern kern, std::atomic<int>* configured, int dev) {
    if (dev < kMaxDevices && configured[dev].load(std::memory_order_acquire)) return ALPHA_MOE_OK;
    CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem));
    if (dev < kMaxDevices) configured[dev].store(1, std::memory_order_release);
    return ALPHA_MOE_OK;
}

// Every fused kernel is launched with programmatic stream serialisation: its CTAs may be scheduled while the kernel
// in front of it in the stream is finishing (this library's quantise / schedule kernels say when), and its first
// statement is the wait for that kernel's completion - so launch latency overlaps the predecessor instead of following it.
template <typename Kern>
int launch_dependent(Kern kern, int grid, int threads, int smem_bytes, int cluster, cudaStream_t stream, const MapSet& maps,
                     const amoe::MoeParams& p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(threads));
    cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    int n = 0;
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
    if (cluster > 1) {
        attrs[n].id = cudaLaunchAttributeClusterDimension;
        attrs[n].val.clusterDim.x = static_cast<unsigned>(cluster);
        attrs[n].val.clusterDim.y = 1;
        attrs[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = static_cast<unsigned>(n);
    CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, maps.w, maps.w2, p));
    return ALPHA_MOE_OK;
}

template <int BMP, int SPC, int EW = (BMP >= 64 ? 2 : 1), bool PEERS = false>
int launch_variant(const MapSet& maps, const amoe::MoeParams& p, int grid, int smem_bytes, int dev, cudaStream_t stream) {
    auto kern = amoe::fused_moe_w8a8_up_down_sm100_kernel<BMP, SPC, EW, PEERS>;
    static std::atomic<int> configured[kMaxDevices];
    if (int rc = ensure_smem_attr(kern, configured, dev)) return rc;
    constexpr int threads = 128 * EW + 128;
    return launch_dependent(kern, grid, threads, smem_bytes, p.ksplit, stream, maps, p);
}

template <int SPC>
int launch_tokmajor(const MapSet& maps, const amoe::MoeParams& p, int grid, int smem_bytes, int dev, cudaStream_t stream) {
    auto kern = amoe::fused_moe_w8a8_up_down_sm100_tokmajor_kernel<SPC>;
    static std::atomic<int> configured[kMaxDevices];
    if (int rc = ensure_smem_attr(kern, configured, dev)) return rc;
    return launch_dependent(kern, grid, amoe::kTmThreads, smem_bytes, 1, stream, maps, p);
}

// Launch of one of the exchange kernels as a programmatic dependent of the kernel in front of it in the stream (its
// first statement is griddepcontrol.wait): its CTAs may be scheduled while that kernel - normally the fused kernel,
// which releases its dependents at entry - is still running.
template <typename... KArgs, typename... Args>
cudaError_t launch_after(void (*kern)(KArgs...), int blocks, int threads, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(static_cast<unsigned>(threads));
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Without a device to ask: GPCs of about 18 SMs, a cluster inside one GPC, one CTA per SM.
// With two CTAs per SM a cluster of an even size fills half as many SMs, and two clusters of an odd size share the
// SMs of one.  (The occupancy calculator cannot be asked: it reports one CTA of these kernels per SM whatever the ring
// size, although two do run side by side; the figures below match what was measured - e.g. 58 units at the DeepSeek
// shard shape with a two-slot ring: clusters of 4 fit (48 us), clusters of 5 do not (60 us).)
void two_per_sm_from_one(ClusterCapacity* c) {
    c->two_per_sm[0] = 0;
    c->two_per_sm[1] = 2 * c->one_per_sm[1];
    for (int ks = 2; ks <= kMaxKsplit; ++ks)
        c->two_per_sm[ks] = ks % 2 == 0 ? c->one_per_sm[ks / 2] : 2 * c->one_per_sm[ks];
}

void model_cluster_capacity(int sms, ClusterCapacity* c) {
    const int gpcs = sms >= 18 ? (sms + 9) / 18 : 1;
    const int per_gpc = sms / gpcs;
    c->one_per_sm[0] = 0;
    c->one_per_sm[1] = sms;
    for (int ks = 2; ks <= kMaxKsplit; ++ks) c->one_per_sm[ks] = gpcs * (per_gpc / ks);
    two_per_sm_from_one(c);
}

int device_facts(int dev, DeviceFacts* out) {
    static DeviceFacts facts[kMaxDevices];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    DeviceFacts local;
    DeviceFacts& f = dev < kMaxDevices ? facts[dev] : local;
    if (!f.status) {
        CUDA_TRY(cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, dev));
        model_cluster_capacity(f.sms, &f.clusters);
        // The driver knows how the SMs are grouped (a cluster lives inside one GPC): ask it, keep the model's figure
        // where it does not answer.  Asked for the narrow weight-major shape with a ring that leaves room for one CTA
        // per SM; the figures for two per SM follow from those.
        auto kern = amoe::fused_moe_w8a8_up_down_sm100_kernel<16, 1>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem) == cudaSuccess) {
            auto ask = [&](int ks, int smem_bytes, int* into) {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(static_cast<unsigned>(ks * 64));
                cfg.blockDim = dim3(256);
                cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
                cudaLaunchAttribute attr;
                attr.id = cudaLaunchAttributeClusterDimension;
                attr.val.clusterDim.x = static_cast<unsigned>(ks);
                attr.val.clusterDim.y = 1;
                attr.val.clusterDim.z = 1;
                cfg.attrs = &attr;
                cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) *into = n;
            };
            for (int ks = 2; ks <= kMaxKsplit; ++ks) ask(ks, kPairDynSmem + 1024, &f.clusters.one_per_sm[ks]);
        }
        two_per_sm_from_one(&f.clusters);
        (void)cudaGetLastError();
        CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&f.status), g_status));
    }
    *out = f;
    return ALPHA_MOE_OK;
}

// Self-test of the bounded wait: warp 0 waits on an mbarrier that nothing ever arrives on, with a limit given by the
// caller; warp 1 waits on a second such barrier with the product's (one second) limit and must be released by the
// CTA's abort flag when warp 0 gives up.  result[0] / result[1] = what the two waits returned (1 = barrier completed).
__global__ void wait_selftest_kernel(amoe::KernelStatus* status, int* result, long long limit_cycles, int where, int iter) {
    __shared__ uint64_t bars[2];
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        amoe::mbar_init(&bars[0], 1);
        amoe::mbar_init(&bars[1], 1);
        abort_flag = 0;
        amoe::fence_mbar_init();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) {
        const bool done = warp == 0 ? amoe::mbar_wait_limit(&bars[0], 0, &abort_flag, status, where, iter, limit_cycles)
                                    : amoe::mbar_wait(&bars[1], 0, &abort_flag, status, where + 1, iter);
        result[warp] = done ? 1 : 0;
    }
}

std::atomic<int> g_ksplit_override{0};     // 0 = automatic; set through alpha_moe_b200_set_ksplit (tuners, tests)

// Clusters of CTAs along K for small batches (narrow tile, one slice per CTA only): the largest cluster size for
// which every (block, slice) unit of the launch still gets its cluster at once.  The capacity tables say how many
// clusters of ks CTAs the device holds at the same time - with the ring the plan arrives at for that ks, which decides
// whether one or two CTAs fit an SM; a launch with more units than that runs in two rounds and loses more than the
// split gains (34 units at the DeepSeek shard shape: clusters of 3 34 us, of 4 49 us).
int choose_ksplit(int block_m, int spc, long long nblocks, int N, int K, int stages, const ClusterCapacity& cap) {
    if (block_m > 32 || spc != 1) return 1;
    const long long units = nblocks * (N / 256);
    const int v = g_ksplit_override.load(std::memory_order_relaxed);
    if (v >= 1 && v <= kMaxKsplit && v <= K / 128) return v;
    for (int ks = kMaxKsplit; ks >= 2; --ks) {
        if (ks > K / 128) continue;
        int depth, bmp, smem_bytes;
        if (plan(K, block_m, stages, spc, ks, &depth, &bmp, &smem_bytes)) continue;
        const int fit = smem_bytes <= kPairDynSmem - 8192 ? cap.two_per_sm[ks] : cap.one_per_sm[ks];
        if (units <= fit) return ks;
    }
    return 1;
}

// Cross-GPU barrier of the fused tensor-parallel path.  flags[r] = rank r's flag array (kMaxTpWorld + 1 words of
// symmetric memory, zero before the first use): word q = last epoch that rank q has announced to r, word kMaxTpWorld =
// r's own epoch counter.  Thread t tells rank t "rank `rank` has reached epoch e" and waits (bounded) until rank t has
// told this rank the same.  The stores are system-scope releases issued after the preceding kernel of the stream has
// completed, so everything that kernel added into the peers' buffers is visible to whoever sees the flag.
struct TpFlags {
    uint32_t* of_rank[amoe::kMaxTpWorld];
};
__global__ void tp_barrier_kernel(TpFlags flags, int world, int rank, amoe::KernelStatus* status, long long limit_cycles) {
    __shared__ uint32_t epoch;
    amoe::griddep_wait();       // launched as a programmatic dependent: the kernel in front must have completed
    uint32_t* mine = flags.of_rank[rank];
    if (threadIdx.x == 0) {
        epoch = mine[amoe::kMaxTpWorld] + 1;
        mine[amoe::kMaxTpWorld] = epoch;
    }
    __syncthreads();
    const int t = threadIdx.x;
    if (t >= world) return;
    const uint32_t e = epoch;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.of_rank[t] + rank), "r"(e) : "memory");
    const long long t0 = clock64();
    for (;;) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + t) : "memory");
        if (static_cast<int32_t>(seen - e) >= 0) return;
        if (clock64() - t0 > limit_cycles) {
            if (atomicCAS(&status->code, amoe::ST_OK, amoe::ST_WAIT_TIMEOUT) == amoe::ST_OK) {
                status->block = rank;
                status->where = 90 + t;          // 90 + the rank that did not arrive
                status->iter = static_cast<int>(e);
            }
            return;
        }
    }
}

// Exchange step of the tensor-parallel small-batch path as one kernel: barrier over the ranks, then every rank sums
// all ranks' partial outputs (plain 16-byte loads from the peers' buffers over NVLink, fp32 sums in rank order, so
// that every rank gets the same bits), writes its own copy of the result and clears its partial buffer of the NEXT
// step.  flags as in tp_barrier_kernel, plus word kMaxTpWorld + 1 = a ticket counter: the last CTA to finish advances
// the epoch, so the epoch a launch reads at its start is stable while it runs (and the kernel replays from a graph).
struct TpExchange {
    const uint4* part[amoe::kMaxTpWorld];
    uint32_t* flags[amoe::kMaxTpWorld];
};
__global__ void __launch_bounds__(256)
tp_exchange_sum_kernel(TpExchange b, uint4* result, uint4* clear_next, int nvec, int nclear, int world, int rank,
                       amoe::KernelStatus* status, long long limit_cycles) {
    __shared__ int arrived;
    amoe::griddep_wait();       // launched as a programmatic dependent: the fused kernel in front must have completed
    uint32_t* mine = b.flags[rank];
    const int t = threadIdx.x;
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(mine + amoe::kMaxTpWorld) + 1;
    if (t == 0) arrived = 1;
    __syncthreads();
    if (t < world) {
        if (blockIdx.x == 0) {
            __threadfence_system();
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(b.flags[t] + rank), "r"(e) : "memory");
        }
        const long long t0 = clock64();
        for (;;) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + t) : "memory");
            if (static_cast<int32_t>(seen - e) >= 0) break;
            if (clock64() - t0 > limit_cycles) {
                arrived = 0;
                if (atomicCAS(&status->code, amoe::ST_OK, amoe::ST_WAIT_TIMEOUT) == amoe::ST_OK) {
                    status->block = rank;
                    status->where = 90 + t;
                    status->iter = static_cast<int>(e);
                }
                break;
            }
        }
    }
    __syncthreads();
    const int stride = gridDim.x * blockDim.x;
    if (arrived) {
        for (int v = blockIdx.x * blockDim.x + t; v < nvec; v += stride) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int r = 0; r < world; ++r) {
                uint4 q;
                asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "l"(b.part[r] + v) : "memory");
                const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[i]));
                    acc[2 * i] += f.x;
                    acc[2 * i + 1] += f.y;
                }
            }
            uint32_t o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                o[i] = *reinterpret_cast<uint32_t*>(&h);
            }
            result[v] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
    for (int v = blockIdx.x * blockDim.x + t; v < nclear; v += stride) clear_next[v] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    if (t == 0) {
        __threadfence();
        const uint32_t ticket = atomicAdd(mine + amoe::kMaxTpWorld + 1, 1u);
        if (ticket == gridDim.x - 1) {
            mine[amoe::kMaxTpWorld + 1] = 0;
            mine[amoe::kMaxTpWorld] = e;
            __threadfence();
        }
    }
}

// All-reduce (sum, bf16, in place) of the ranks' partial outputs for large batches, as one kernel over peer-mapped
// buffers: barrier; every rank sums ITS 1/world slice over all ranks (16-byte loads over NVLink, fp32, rank order) and
// writes it back into its own buffer; second barrier; every rank copies the other slices from their owners.  Each
// rank reads 2 (world-1)/world of the payload over NVLink, like a ring or two-shot collective, but with plain loads
// and two flag barriers instead of a protocol.  Flags and epochs as in tp_exchange_sum_kernel (two epochs per call);
// the "this rank has finished its slice" signal is sent by the last CTA to finish phase 1 (ticket counter).
template <int UNROLL>
__device__ __forceinline__ bool tp_wait_all(uint32_t* mine, int world, uint32_t e, int rank, amoe::KernelStatus* status,
                                            long long limit_cycles, int where_base) {
    __shared__ int arrived_s;
    const int t = threadIdx.x;
    if (t == 0) arrived_s = 1;
    __syncthreads();
    if (t < world) {
        const long long t0 = clock64();
        for (;;) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + t) : "memory");
            if (static_cast<int32_t>(seen - e) >= 0) break;
            if (clock64() - t0 > limit_cycles) {
                arrived_s = 0;
                if (atomicCAS(&status->code, amoe::ST_OK, amoe::ST_WAIT_TIMEOUT) == amoe::ST_OK) {
                    status->block = rank;
                    status->where = where_base + t;
                    status->iter = static_cast<int>(e);
                }
                break;
            }
        }
    }
    __syncthreads();
    return arrived_s != 0;
}
__device__ __forceinline__ void tp_signal_all(const TpExchange& b, int world, int rank, uint32_t e) {
    if (threadIdx.x < world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(b.flags[threadIdx.x] + rank), "r"(e) : "memory");
    }
}
__device__ __forceinline__ uint4 ld_cg_v4(const uint4* p) {
    uint4 q;
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "l"(p) : "memory");
    return q;
}
__global__ void __launch_bounds__(256)
tp_allreduce_kernel(TpExchange b, int nvec, int world, int rank, amoe::KernelStatus* status, long long limit_cycles,
                    int gather) {
    amoe::griddep_wait();       // launched as a programmatic dependent: the fused kernel in front must have completed
    uint32_t* mine = b.flags[rank];
    uint32_t* ticket = mine + amoe::kMaxTpWorld + 1;
    const int t = threadIdx.x;
    const uint32_t e0 = *reinterpret_cast<volatile uint32_t*>(mine + amoe::kMaxTpWorld);
    uint4* own = const_cast<uint4*>(b.part[rank]);
    if (blockIdx.x == 0) tp_signal_all(b, world, rank, e0 + 1);              // my fused kernel has finished (stream order)
    bool ok = tp_wait_all<0>(mine, world, e0 + 1, rank, status, limit_cycles, 90);
    const int per = (nvec + world - 1) / world;
    const int stride = gridDim.x * blockDim.x;
    if (ok) {
        // phase 1: my slice, summed over all ranks, two vectors per thread and step
        const int lo = rank * per, hi = min(nvec, lo + per);
        for (int v = lo + blockIdx.x * blockDim.x + t; v < hi; v += 2 * stride) {
            const int v2 = v + stride;
            uint4 a[amoe::kMaxTpWorld], c[amoe::kMaxTpWorld];
#pragma unroll
            for (int r = 0; r < amoe::kMaxTpWorld; ++r) {
                if (r < world) {
                    a[r] = ld_cg_v4(b.part[r] + v);
                    if (v2 < hi) c[r] = ld_cg_v4(b.part[r] + v2);
                }
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (half == 1 && v2 >= hi) break;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < amoe::kMaxTpWorld; ++r) {
                    if (r < world) {
                        const uint4 q = half ? c[r] : a[r];
                        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[i]));
                            acc[2 * i] += f.x;
                            acc[2 * i + 1] += f.y;
                        }
                    }
                }
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                    o[i] = *reinterpret_cast<uint32_t*>(&h);
                }
                own[half ? v2 : v] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    }
    // the last CTA of this rank to get here tells the peers that the slice is complete
    __shared__ int last_s;
    __syncthreads();
    if (t == 0) {
        __threadfence();
        last_s = atomicAdd(ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (last_s) tp_signal_all(b, world, rank, e0 + 2);
    ok = tp_wait_all<1>(mine, world, e0 + 2, rank, status, limit_cycles, 100) && ok;
    if (ok && gather) {
        // phase 2 (all-reduce only; a reduce-scatter stops at the barrier above, after which no rank reads a peer's
        // buffer any more): the other ranks' finished slices, four vectors per thread and step
        for (int q = 1; q < world; ++q) {
            const int r = (rank + q) % world;
            const int lo = r * per, hi = min(nvec, lo + per);
            const uint4* src = b.part[r];
            for (int v = lo + blockIdx.x * blockDim.x + t; v < hi; v += 4 * stride) {
                uint4 x0 = ld_cg_v4(src + v), x1, x2, x3;
                if (v + stride < hi) x1 = ld_cg_v4(src + v + stride);
                if (v + 2 * stride < hi) x2 = ld_cg_v4(src + v + 2 * stride);
                if (v + 3 * stride < hi) x3 = ld_cg_v4(src + v + 3 * stride);
                own[v] = x0;
                if (v + stride < hi) own[v + stride] = x1;
                if (v + 2 * stride < hi) own[v + 2 * stride] = x2;
                if (v + 3 * stride < hi) own[v + 3 * stride] = x3;
            }
        }
    }
    __syncthreads();
    if (t == 0) {
        __threadfence();
        if (atomicAdd(ticket, 1u) == 2 * gridDim.x - 1) {      // every CTA has passed both phases
            *ticket = 0;
            mine[amoe::kMaxTpWorld] = e0 + 2;
            __threadfence();
        }
    }
}

int launch_fused(const void* x, const float* x_scale, const void* w, const float* w_scale, const void* w2,
                 const float* w2_scale, void* const* outs, int tp_world, int tp_rank, const int32_t* sorted_token_ids,
                 const int32_t* expert_ids, const int32_t* num_tokens_post_padded, const float* topk_weights, int top_k,
                 int M, int K, int N, int num_experts, int sorted_num, int block_m, int block_n, int warp_n, int stages,
                 float scaling_factor, void* stream) {
    if (!x || !x_scale || !w || !w_scale || !w2 || !w2_scale || !outs || !sorted_token_ids || !expert_ids ||
        !num_tokens_post_padded || !topk_weights)
        return fail(ALPHA_MOE_E_ARG, "null pointer argument");
    if (tp_world < 1 || tp_world > amoe::kMaxTpWorld || tp_rank < 0 || tp_rank >= tp_world)
        return fail(ALPHA_MOE_E_ARG, "tp_world must be in 1..%d and 0 <= tp_rank < tp_world (got %d, %d)",
                    amoe::kMaxTpWorld, tp_world, tp_rank);
    for (int r = 0; r < tp_world; ++r)
        if (!outs[r]) return fail(ALPHA_MOE_E_ARG, "null pointer argument (out of rank %d)", r);
    if (tp_world > 1 && block_m > 64)
        return fail(ALPHA_MOE_E_ARG, "the fused tensor-parallel exchange serves small batches: block_m <= 64 (got %d); "
                                     "larger blocks run the plain operator followed by an all-reduce", block_m);
    void* out = outs[tp_rank];
    if (M <= 0) return fail(ALPHA_MOE_E_ARG, "x must have at least one row (M=%d)", M);
    if (K <= 0 || K % 128 != 0) return fail(ALPHA_MOE_E_ARG, "K dimension must be a multiple of 128 (K=%d)", K);
    if (N <= 0 || N % 256 != 0) return fail(ALPHA_MOE_E_ARG, "N must be a multiple of 256 (N=%d)", N);
    if (num_experts <= 0 || top_k <= 0 || sorted_num <= 0)
        return fail(ALPHA_MOE_E_ARG, "num_experts, top_k and sorted_num must be positive");
    if (!((block_n == 64 && warp_n == 4) || (block_n == 32 && warp_n == 8)))
        return fail(ALPHA_MOE_E_ARG, "(block_n, warp_n) must be (64,4) or (32,8), got (%d,%d)", block_n, warp_n);
    if (stages < 1 || stages > 5) return fail(ALPHA_MOE_E_ARG, "stages must be in 1..5, got %d", stages);
    if (block_m < 8 || block_m > 128 || block_m % 8 != 0)
        return fail(ALPHA_MOE_E_ARG, "block_m must be a multiple of 8 in 8..128, got %d", block_m);
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(w2) | reinterpret_cast<uintptr_t>(x)) & 15)
        return fail(ALPHA_MOE_E_ARG, "x, w and w2 must be 16-byte aligned");
    // the token-major kernels accumulate with 16-byte vector reductions, the others with 4-byte ones
    for (int r = 0; r < tp_world; ++r)
        if (reinterpret_cast<uintptr_t>(outs[r]) & (token_major(block_m) ? 15 : 3))
            return fail(ALPHA_MOE_E_ARG, "out must be %d-byte aligned for block_m=%d", token_major(block_m) ? 16 : 4, block_m);
    if (static_cast<long long>(M) * top_k > 0x7FFFFFFFLL) return fail(ALPHA_MOE_E_ARG, "M*top_k overflows int32");

    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    DeviceFacts facts;
    if (int rc = device_facts(dev, &facts)) return rc;

    // block_n = 64 asks for the wide variant: one CTA owns two 128-column slices of the intermediate
    // dimension (one reduction per token and expert instead of two); it needs an even slice count.
    const int spc = (block_n == 64 && (N / 256) % 2 == 0) ? 2 : 1;
    // Live blocks never exceed the number of assignments, so no more CTAs than that are launched.
    long long nblocks = (static_cast<long long>(sorted_num) + block_m - 1) / block_m;
    if (nblocks > static_cast<long long>(M) * top_k) nblocks = static_cast<long long>(M) * top_k;
    const int ksplit = choose_ksplit(block_m, spc, nblocks, N, K, stages, facts.clusters);
    int depth, bmp, smem_bytes;
    if (int rc = plan(K, block_m, stages, spc, ksplit, &depth, &bmp, &smem_bytes)) return rc;

    MapSet maps;
    if (int rc = get_maps(dev, w, w2, num_experts, N, K, &maps)) return rc;

    amoe::MoeParams p;
    p.x = static_cast<const uint8_t*>(x);
    p.x_scale = x_scale;
    p.w_scale = w_scale;
    p.w2_scale = w2_scale;
    p.out = static_cast<__nv_bfloat16*>(out);
    p.tp_world = tp_world;
    for (int i = 0; i < amoe::kMaxTpWorld - 1; ++i)       // the peers, starting behind this rank so that traffic spreads
        p.out_more[i] = i + 1 < tp_world ? static_cast<__nv_bfloat16*>(outs[(tp_rank + 1 + i) % tp_world]) : nullptr;
    p.sorted_token_ids = sorted_token_ids;
    p.expert_ids = expert_ids;
    p.num_tokens_post_padded = num_tokens_post_padded;
    p.topk_weights = topk_weights;
    p.top_k = top_k;
    p.M = M;
    p.K = K;
    p.N = N;
    p.E = num_experts;
    p.sorted_num = sorted_num;
    p.block_m = block_m;
    p.stages = depth;
    p.ksplit = ksplit;
    p.scaling = scaling_factor;
    p.status = facts.status;

    const long long grid = nblocks * (N / 256 / spc) * ksplit;
    if (grid > 0x7FFFFFFFLL) return fail(ALPHA_MOE_E_ARG, "grid too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int g = static_cast<int>(grid);
    // A 64-wide tile with a ring of at most two slots runs the single-warpgroup shape, two CTAs per SM
    // (227 KB per SM less 1 KB reserved per CTA leaves 113 KB of dynamic shared memory for each).
    const bool pair64 = bmp == 64 && depth <= 2 && smem_bytes <= kPairDynSmem;
    if (token_major(block_m))
        return spc == 1 ? launch_tokmajor<1>(maps, p, g, smem_bytes, dev, st)
                        : launch_tokmajor<2>(maps, p, g, smem_bytes, dev, st);
    if (tp_world > 1) {       // the form that adds into the peers' buffers: one shape per tile width
        if (spc == 1) {
            switch (bmp) {
                case 16: return launch_variant<16, 1, 1, true>(maps, p, g, smem_bytes, dev, st);
                case 32: return launch_variant<32, 1, 1, true>(maps, p, g, smem_bytes, dev, st);
                default: return launch_variant<64, 1, 2, true>(maps, p, g, smem_bytes, dev, st);
            }
        }
        switch (bmp) {
            case 16: return launch_variant<16, 2, 1, true>(maps, p, g, smem_bytes, dev, st);
            case 32: return launch_variant<32, 2, 1, true>(maps, p, g, smem_bytes, dev, st);
            default: return launch_variant<64, 2, 2, true>(maps, p, g, smem_bytes, dev, st);
        }
    }
    if (spc == 1) {
        switch (bmp) {
            case 16: return launch_variant<16, 1>(maps, p, g, smem_bytes, dev, st);
            case 32: return launch_variant<32, 1>(maps, p, g, smem_bytes, dev, st);
            default: return pair64 ? launch_variant<64, 1, 1>(maps, p, g, smem_bytes, dev, st)
                                   : launch_variant<64, 1>(maps, p, g, smem_bytes, dev, st);
        }
    }
    switch (bmp) {
        case 16: return launch_variant<16, 2>(maps, p, g, smem_bytes, dev, st);
        case 32: return launch_variant<32, 2>(maps, p, g, smem_bytes, dev, st);
        default: return pair64 ? launch_variant<64, 2, 1>(maps, p, g, smem_bytes, dev, st)
                               : launch_variant<64, 2>(maps, p, g, smem_bytes, dev, st);
    }
}

}  // namespace

extern "C" {

int alpha_moe_b200_fused_moe_w8a8_up_down(const void* x, const float* x_scale, const void* w, const float* w_scale,
                                          const void* w2, const float* w2_scale, void* out,
                                          const int32_t* sorted_token_ids, const int32_t* expert_ids,
                                          const int32_t* num_tokens_post_padded, const float* topk_weights, int top_k,
                                          int M, int K, int N, int num_experts, int sorted_num, int block_m,
                                          int block_n, int warp_n, int stages, float scaling_factor, void* stream) {
    if (!out) return fail(ALPHA_MOE_E_ARG, "null pointer argument");
    void* outs[1] = {out};
    return launch_fused(x, x_scale, w, w_scale, w2, w2_scale, outs, 1, 0, sorted_token_ids, expert_ids,
                        num_tokens_post_padded, topk_weights, top_k, M, K, N, num_experts, sorted_num, block_m, block_n,
                        warp_n, stages, scaling_factor, stream);
}

int alpha_moe_b200_fused_moe_w8a8_up_down_tp(const void* x, const float* x_scale, const void* w, const float* w_scale,
                                             const void* w2, const float* w2_scale, void* const* outs, int tp_world,
                                             int tp_rank, const int32_t* sorted_token_ids, const int32_t* expert_ids,
                                             const int32_t* num_tokens_post_padded, const float* topk_weights, int top_k,
                                             int M, int K, int N, int num_experts, int sorted_num, int block_m,
                                             int block_n, int warp_n, int stages, float scaling_factor, void* stream) {
    return launch_fused(x, x_scale, w, w_scale, w2, w2_scale, outs, tp_world, tp_rank, sorted_token_ids, expert_ids,
                        num_tokens_post_padded, topk_weights, top_k, M, K, N, num_experts, sorted_num, block_m, block_n,
                        warp_n, stages, scaling_factor, stream);
}

int alpha_moe_b200_tp_barrier(void* const* flags, int tp_world, int tp_rank, int timeout_ms, void* stream) {
    if (!flags) return fail(ALPHA_MOE_E_ARG, "flags is null");
    if (tp_world < 1 || tp_world > amoe::kMaxTpWorld || tp_rank < 0 || tp_rank >= tp_world)
        return fail(ALPHA_MOE_E_ARG, "tp_world must be in 1..%d and 0 <= tp_rank < tp_world (got %d, %d)",
                    amoe::kMaxTpWorld, tp_world, tp_rank);
    if (timeout_ms < 1 || timeout_ms > 2000) return fail(ALPHA_MOE_E_ARG, "timeout_ms must be in 1..2000, got %d", timeout_ms);
    TpFlags f;
    for (int r = 0; r < amoe::kMaxTpWorld; ++r) {
        f.of_rank[r] = r < tp_world ? static_cast<uint32_t*>(flags[r]) : nullptr;
        if (r < tp_world && (!flags[r] || (reinterpret_cast<uintptr_t>(flags[r]) & 3)))
            return fail(ALPHA_MOE_E_ARG, "flag array of rank %d is null or misaligned", r);
    }
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    DeviceFacts facts;
    if (int rc = device_facts(dev, &facts)) return rc;
    const long long limit = static_cast<long long>(timeout_ms) * 2000000LL;      // about 2 GHz
    CUDA_TRY(launch_after(tp_barrier_kernel, 1, 32, static_cast<cudaStream_t>(stream), f, tp_world, tp_rank, facts.status, limit));
    return ALPHA_MOE_OK;
}

int alpha_moe_b200_tp_exchange_sum(void* const* partials, void* result, void* clear_next, long long count, long long clear_count,
                                   void* const* flags, int tp_world, int tp_rank, int timeout_ms, void* stream) {
    if (!partials || !result || !flags) return fail(ALPHA_MOE_E_ARG, "null pointer argument");
    if (tp_world < 1 || tp_world > amoe::kMaxTpWorld || tp_rank < 0 || tp_rank >= tp_world)
        return fail(ALPHA_MOE_E_ARG, "tp_world must be in 1..%d and 0 <= tp_rank < tp_world (got %d, %d)",
                    amoe::kMaxTpWorld, tp_world, tp_rank);
    if (timeout_ms < 1 || timeout_ms > 2000) return fail(ALPHA_MOE_E_ARG, "timeout_ms must be in 1..2000, got %d", timeout_ms);
    if (count <= 0 || count % 8 != 0 || clear_count < 0 || clear_count % 8 != 0 || count > 0x3FFFFFFFLL * 8 ||
        clear_count > 0x3FFFFFFFLL * 8)
        return fail(ALPHA_MOE_E_ARG, "count and clear_count are bf16 element counts, multiples of 8 (got %lld, %lld)", count,
                    clear_count);
    if (clear_count > 0 && !clear_next) return fail(ALPHA_MOE_E_ARG, "clear_next is null");
    TpExchange b;
    for (int r = 0; r < amoe::kMaxTpWorld; ++r) {
        b.part[r] = r < tp_world ? static_cast<const uint4*>(partials[r]) : nullptr;
        b.flags[r] = r < tp_world ? static_cast<uint32_t*>(flags[r]) : nullptr;
        if (r < tp_world && (!partials[r] || !flags[r] || (reinterpret_cast<uintptr_t>(partials[r]) & 15) ||
                             (reinterpret_cast<uintptr_t>(flags[r]) & 3)))
            return fail(ALPHA_MOE_E_ARG, "partial buffer or flag array of rank %d is null or misaligned", r);
    }
    if ((reinterpret_cast<uintptr_t>(result) & 15) || (reinterpret_cast<uintptr_t>(clear_next) & 15))
        return fail(ALPHA_MOE_E_ARG, "result and clear_next must be 16-byte aligned");
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    DeviceFacts facts;
    if (int rc = device_facts(dev, &facts)) return rc;
    const int nvec = static_cast<int>(count / 8), nclear = static_cast<int>(clear_count / 8);
    int blocks = (std::max(nvec, nclear) + 255) / 256;
    blocks = std::max(1, std::min(blocks, facts.sms));
    const long long limit = static_cast<long long>(timeout_ms) * 2000000LL;
    CUDA_TRY(launch_after(tp_exchange_sum_kernel, blocks, 256, static_cast<cudaStream_t>(stream), b, static_cast<uint4*>(result),
                          static_cast<uint4*>(clear_next), nvec, nclear, tp_world, tp_rank, facts.status, limit));
    return ALPHA_MOE_OK;
}

namespace {
int tp_reduce(void* const* bufs, long long count, void* const* flags, int tp_world, int tp_rank, int timeout_ms,
              void* stream, int gather);
}

int alpha_moe_b200_tp_allreduce(void* const* bufs, long long count, void* const* flags, int tp_world, int tp_rank,
                                int timeout_ms, void* stream) {
    return tp_reduce(bufs, count, flags, tp_world, tp_rank, timeout_ms, stream, 1);
}

int alpha_moe_b200_tp_reduce_scatter(void* const* bufs, long long count, void* const* flags, int tp_world, int tp_rank,
                                     int timeout_ms, void* stream) {
    return tp_reduce(bufs, count, flags, tp_world, tp_rank, timeout_ms, stream, 0);
}

namespace {
int tp_reduce(void* const* bufs, long long count, void* const* flags, int tp_world, int tp_rank, int timeout_ms,
              void* stream, int gather) {
    if (!bufs || !flags) return fail(ALPHA_MOE_E_ARG, "null pointer argument");
    if (tp_world < 1 || tp_world > amoe::kMaxTpWorld || tp_rank < 0 || tp_rank >= tp_world)
        return fail(ALPHA_MOE_E_ARG, "tp_world must be in 1..%d and 0 <= tp_rank < tp_world (got %d, %d)",
                    amoe::kMaxTpWorld, tp_world, tp_rank);
    if (timeout_ms < 1 || timeout_ms > 2000) return fail(ALPHA_MOE_E_ARG, "timeout_ms must be in 1..2000, got %d", timeout_ms);
    if (count <= 0 || count % 8 != 0 || count > 0x3FFFFFFFLL * 8)
        return fail(ALPHA_MOE_E_ARG, "count is a bf16 element count, a multiple of 8 (got %lld)", count);
    TpExchange b;
    for (int r = 0; r < amoe::kMaxTpWorld; ++r) {
        b.part[r] = r < tp_world ? static_cast<const uint4*>(bufs[r]) : nullptr;
        b.flags[r] = r < tp_world ? static_cast<uint32_t*>(flags[r]) : nullptr;
        if (r < tp_world && (!bufs[r] || !flags[r] || (reinterpret_cast<uintptr_t>(bufs[r]) & 15) ||
                             (reinterpret_cast<uintptr_t>(flags[r]) & 3)))
            return fail(ALPHA_MOE_E_ARG, "buffer or flag array of rank %d is null or misaligned", r);
    }
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    DeviceFacts facts;
    if (int rc = device_facts(dev, &facts)) return rc;
    const int nvec = static_cast<int>(count / 8);
    const int per = (nvec + tp_world - 1) / tp_world;
    // every CTA must be resident at once (all of them wait for the peers): at most one per SM
    const int blocks = std::max(1, std::min((per + 511) / 512, facts.sms));      // (two per SM measured the same)
    const long long limit = static_cast<long long>(timeout_ms) * 2000000LL;
    CUDA_TRY(launch_after(tp_allreduce_kernel, blocks, 256, static_cast<cudaStream_t>(stream), b, nvec, tp_world, tp_rank,
                          facts.status, limit, gather));
    return ALPHA_MOE_OK;
}
}  // namespace

int alpha_moe_b200_selftest_wait_timeout(int limit_cycles, int where, int iter, int32_t* result2, void* stream) {
    if (!result2) return fail(ALPHA_MOE_E_ARG, "result2 is null");
    if (limit_cycles < 1000 || limit_cycles > 200000000)
        return fail(ALPHA_MOE_E_ARG, "limit_cycles must be in 1000..200000000 (about 0.1 s), got %d", limit_cycles);
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    DeviceFacts facts;
    if (int rc = device_facts(dev, &facts)) return rc;
    wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(facts.status, result2, limit_cycles, where, iter);
    CUDA_TRY(cudaGetLastError());
    return ALPHA_MOE_OK;
}

int alpha_moe_b200_set_ksplit(int ksplit) {
    if (ksplit < 0 || ksplit > kMaxKsplit)
        return fail(ALPHA_MOE_E_ARG, "ksplit must be 0 (automatic) or 1..8 CTAs per cluster, got %d", ksplit);
    g_ksplit_override.store(ksplit, std::memory_order_relaxed);
    return ALPHA_MOE_OK;
}

int alpha_moe_b200_read_status(int32_t* out4, int reset) {
    if (!out4) return fail(ALPHA_MOE_E_ARG, "out4 is null");
    CUDA_TRY(cudaDeviceSynchronize());
    amoe::KernelStatus h;
    CUDA_TRY(cudaMemcpyFromSymbol(&h, g_status, sizeof(h)));
    out4[0] = h.code;
    out4[1] = h.block;
    out4[2] = h.where;
    out4[3] = h.iter;
    if (reset) {
        amoe::KernelStatus z = {0, 0, 0, 0};
        CUDA_TRY(cudaMemcpyToSymbol(g_status, &z, sizeof(z)));
    }
    return ALPHA_MOE_OK;
}

int alpha_moe_b200_plan(int K, int N, int block_m, int block_n, int stages, int num_blocks, int num_sms,
                        int32_t* out6) {
    if (!out6) return fail(ALPHA_MOE_E_ARG, "out6 is null");
    if (K <= 0 || K % 128 != 0) return fail(ALPHA_MOE_E_ARG, "K dimension must be a multiple of 128 (K=%d)", K);
    if (N <= 0 || N % 256 != 0) return fail(ALPHA_MOE_E_ARG, "N must be a multiple of 256 (N=%d)", N);
    if (block_m < 8 || block_m > 128 || block_m % 8 != 0) return fail(ALPHA_MOE_E_ARG, "bad block_m %d", block_m);
    if (block_n != 32 && block_n != 64) return fail(ALPHA_MOE_E_ARG, "block_n must be 32 or 64, got %d", block_n);
    if (stages < 1 || stages > 5) return fail(ALPHA_MOE_E_ARG, "stages must be in 1..5, got %d", stages);
    if (num_blocks <= 0 || num_sms < 0) return fail(ALPHA_MOE_E_ARG, "num_blocks must be positive, num_sms >= 0");
    const int spc = (block_n == 64 && (N / 256) % 2 == 0) ? 2 : 1;
    ClusterCapacity clusters;
    if (num_sms == 0) {           // the current device, as a launch would see it
        int dev = 0;
        CUDA_TRY(cudaGetDevice(&dev));
        DeviceFacts facts;
        if (int rc = device_facts(dev, &facts)) return rc;
        clusters = facts.clusters;
    } else {
        model_cluster_capacity(num_sms, &clusters);
    }
    const int ksplit = choose_ksplit(block_m, spc, num_blocks, N, K, stages, clusters);
    int depth, bmp, smem_bytes;
    if (int rc = plan(K, block_m, stages, spc, ksplit, &depth, &bmp, &smem_bytes)) return rc;
    out6[0] = depth;
    out6[1] = bmp;
    out6[2] = smem_bytes;
    out6[3] = spc;
    out6[4] = ksplit;
    out6[5] = token_major(block_m) ? 1 : 0;
    return ALPHA_MOE_OK;
}

int alpha_moe_b200_fused_experts(void* hidden_states, void* x_fp8, float* x_scale, const void* w,
                                 const float* w_scale, const void* w2, const float* w2_scale,
                                 const int32_t* topk_ids, const float* topk_weights, int top_k, int M, int K, int N,
                                 int num_experts, int32_t* sorted_token_ids, int32_t* expert_ids,
                                 int32_t* num_tokens_post_padded, void* align_workspace, int block_m, int block_n,
                                 int warp_n, int stages, float scaling_factor, void* stream) {
    if (!hidden_states || !x_fp8 || !x_scale || !topk_ids || !sorted_token_ids || !expert_ids || !num_tokens_post_padded)
        return fail(ALPHA_MOE_E_ARG, "null pointer argument");
    if (M <= 0 || top_k <= 0 || num_experts <= 0) return fail(ALPHA_MOE_E_ARG, "M, top_k and num_experts must be positive");
    if (block_m < 8 || block_m > 128 || block_m % 8 != 0) return fail(ALPHA_MOE_E_ARG, "bad block_m %d", block_m);
    const long long numel = static_cast<long long>(M) * top_k;
    const long long sorted_num = numel + static_cast<long long>(num_experts) * (block_m - 1);
    if (sorted_num > 0x7FFFFFFFLL) return fail(ALPHA_MOE_E_ARG, "schedule too long for int32");
    // extra/sglang.patch:30-31: quantise, then clear the buffer the layer accumulates into; :33-35: the schedule
    // (one launch for both when the schedule fits one CTA)
    if (int rc = alpha_moe_b200_quant_and_align(hidden_states, x_fp8, x_scale, M, K, 1, topk_ids, top_k, num_experts,
                                                block_m, sorted_token_ids, expert_ids, num_tokens_post_padded,
                                                align_workspace, stream))
        return rc;
    // :38-40
    return alpha_moe_b200_fused_moe_w8a8_up_down(x_fp8, x_scale, w, w_scale, w2, w2_scale, hidden_states, sorted_token_ids,
                                                 expert_ids, num_tokens_post_padded, topk_weights, top_k, M, K, N,
                                                 num_experts, static_cast<int>(sorted_num), block_m, block_n, warp_n,
                                                 stages, scaling_factor, stream);
}


const char* alpha_moe_b200_last_error(void) { return g_last_error.c_str(); }
const char* alpha_moe_b200_version(void) { return "alpha_moe_b200 0.1 (sm_100a)"; }

}  // extern "C"
