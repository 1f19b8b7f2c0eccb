// C ABI of the B200 batch SM120 SASS codec: context, kernels and launchers.
//
// Kernels are one thread per instruction word over a grid-stride loop.  A warp reads 32
// consecutive 16-byte words (512 contiguous bytes) and writes 32 consecutive entries of
// every output plane, so all global traffic is coalesced and uses streaming hints.  The
// per-word table lookups are data dependent and diverge between lanes, so the hot part of
// the ISA table (about 215 KB) is staged into shared memory once per CTA by persistent
// CTAs (one per SM, 1024 threads); small batches use a variant that reads the table through
// the read-only global path instead of paying for the staging.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <type_traits>
#include <vector>

#include "../../include/cubit_b200.h"
#include "codec_core.cuh"
#include "elf_text.hpp"
#include "flat_table.hpp"
#include "sass_text.hpp"
#include "isa_table.hpp"

using namespace cubit;

// ---- kernels -----------------------------------------------------------------------------

namespace {

constexpr int kBlock = 256;          // table in global memory
constexpr int kBlockShared = 1024;   // table staged in shared memory, one CTA per SM
constexpr uint64_t kSharedMinWords = 1u << 17;   // below this the staging copy is not worth it
enum { CNT_DECODED = 0, CNT_REJECTED, CNT_TIE, CNT_EXACT, CNT_MISMATCH, CNT_WORDS };

// Copies the kernel's window of the blob into dynamic shared memory, by the whole CTA: words
// [begin, end) for HotShared / HotSharedEnc, the roundtrip kernel's two ranges for HotSharedRT.
template <class HOT>
__device__ __forceinline__ void stage_table(const FlatView&, uint32_t, uint32_t) {}
__device__ __forceinline__ void stage_range(const FlatView& t, uint32_t begin, uint32_t end) {
    const uint4* src = reinterpret_cast<const uint4*>(t.cold + begin);
    const uint32_t quads = (end - begin) / 4;
    for (uint32_t i = threadIdx.x; i < quads; i += blockDim.x) cb_table_smem[i] = __ldg(src + i);
    __syncthreads();
}
template <>
__device__ __forceinline__ void stage_table<HotShared>(const FlatView& t, uint32_t begin, uint32_t end) { stage_range(t, begin, end); }
template <>
__device__ __forceinline__ void stage_table<HotSharedEnc>(const FlatView& t, uint32_t begin, uint32_t end) { stage_range(t, begin, end); }
template <>
__device__ __forceinline__ void stage_table<HotSharedRT>(const FlatView& t, uint32_t, uint32_t) {
    const uint4* src = reinterpret_cast<const uint4*>(t.cold);
    const uint32_t quads_a = t.at.sel_words / 4, first_b = t.at.rt[0] / 4, quads_b = (t.at.total_words - t.at.rt[0]) / 4;
    for (uint32_t i = threadIdx.x; i < quads_a; i += blockDim.x) cb_table_smem[i] = __ldg(src + i);
    for (uint32_t i = threadIdx.x; i < quads_b; i += blockDim.x) cb_table_smem[quads_a + i] = __ldg(src + first_b + i);
    __syncthreads();
}

// Adds per-thread tallies into the launch's counters: warp reduce, then one shared atomic
// per warp, then one global atomic per block.
template <int N>
__device__ __forceinline__ void block_tally(const uint32_t (&mine)[N], const int (&which)[N],
                                            unsigned long long* counters) {
    __shared__ uint32_t s_acc[CNT_WORDS];
    if (threadIdx.x < CNT_WORDS) s_acc[threadIdx.x] = 0;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < N; ++k) {
        const uint32_t w = __reduce_add_sync(0xFFFFFFFFu, mine[k]);
        if ((threadIdx.x & 31) == 0 && w) atomicAdd(&s_acc[which[k]], w);
    }
    __syncthreads();
    if (threadIdx.x < CNT_WORDS && s_acc[threadIdx.x])
        atomicAdd(&counters[threadIdx.x], (unsigned long long)s_acc[threadIdx.x]);
}

// WIDE: the table has leaves of more than 16 classes (the SM120 table has none; its kernels leave that path out).
// COUNT: the caller wants the counters (launches without them leave the per-word tallies out).
// IDX is the type of the word index: uint32_t when the batch allows it (then every plane
// address is one 32 x 32 + 64 bit multiply-add from a plane base that is the same for the
// whole grid), uint64_t otherwise.  The next word of a thread is loaded before the current one
// is decoded, so its latency hides behind the table walk.
template <class HOT, class IDX, bool WIDE, bool COUNT>
__global__ void __launch_bounds__(std::is_same<HOT, HotGlobal>::value ? kBlock : kBlockShared, 1)
decode_kernel(FlatView tg, const uint4* __restrict__ words, uint64_t n64, uint16_t* __restrict__ form,
              uint32_t* __restrict__ slots, uint64_t slot_stride, uint32_t* __restrict__ ctrl,
              unsigned long long* counters) {
    stage_table<HOT>(tg, 0, tg.at.hot_words);
    const FlatView& t = tg;
    uint32_t n_ok = 0, n_tie = 0;
    const IDX n = (IDX)n64;
    const IDX step = (IDX)gridDim.x * (IDX)blockDim.x;
    const IDX first = (IDX)blockIdx.x * (IDX)blockDim.x + (IDX)threadIdx.x;
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (first < n) w = __ldcs(words + first);
    for (IDX i = first; i < n; i += step) {
        uint4 next = w;
        if (n - i > step) next = __ldcs(words + (i + step));
        uint32_t f, c, s[8];
        decode_word<HOT, WIDE>(t, w.x, w.y, w.z, w.w, &f, s, &c);
        __stcs(form + i, (uint16_t)f);
#pragma unroll
        for (int k = 0; k < 8; ++k) __stcs(slots + (uint64_t)k * slot_stride + i, s[k]);
        __stcs(ctrl + i, c);
        if (COUNT) {
            n_ok += (c >> 30) == ST_OK;
            n_tie += (c >> 28) & 1u;
        }
        w = next;
    }
    if (COUNT) {
        // Rejected words are the rest of this thread's share of the batch.
        const uint32_t seen = first < n ? (uint32_t)((n - first + step - 1) / step) : 0u;
        const uint32_t tally[3] = {n_ok, seen - n_ok, n_tie};
        const int which[3] = {CNT_DECODED, CNT_REJECTED, CNT_TIE};
        block_tally(tally, which, counters);
    }
}

// Two records per thread and trip, so that twenty loads are in flight before the first is used
// (measured: one record 78.9, two 84.4, three 80.9 Ginsn/s).  When every plane is 8-byte aligned
// (even stride, aligned bases) a thread takes two neighbouring records with 64-bit loads, which
// halves the number of load instructions; otherwise the two records are a grid stride apart.
template <class HOT>
__global__ void __launch_bounds__(std::is_same<HOT, HotGlobal>::value ? kBlock : kBlockShared)
encode_kernel(FlatView tg, const uint16_t* __restrict__ form, const uint32_t* __restrict__ slots,
              uint64_t slot_stride, const uint32_t* __restrict__ ctrl, uint64_t n, uint4* __restrict__ words, int paired) {
    // The encode kernel stages its own window: deposit and variant records.
    stage_table<HOT>(tg, tg.at.enc, tg.at.enc_end);
    const FlatView& t = tg;
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (paired) {
        const uint64_t pairs = n / 2;
        for (uint64_t p = tid; p < pairs; p += step) {
            uint32_t a[8], b[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint2 v = __ldcs(reinterpret_cast<const uint2*>(slots + (uint64_t)k * slot_stride) + p);
                a[k] = v.x; b[k] = v.y;
            }
            const uint32_t ff = __ldcs(reinterpret_cast<const uint32_t*>(form) + p);
            const uint2 cc = __ldcs(reinterpret_cast<const uint2*>(ctrl) + p);
            uint4 w;
            encode_record<HOT, HOT>(t, ff & 0xFFFFu, a, cc.x, &w.x, &w.y, &w.z, &w.w);
            __stcs(words + 2 * p, w);
            encode_record<HOT, HOT>(t, ff >> 16, b, cc.y, &w.x, &w.y, &w.z, &w.w);
            __stcs(words + 2 * p + 1, w);
        }
        if ((n & 1) && tid == 0) {   // the odd record at the end
            const uint64_t j = n - 1;
            uint32_t a[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) a[k] = __ldcs(slots + (uint64_t)k * slot_stride + j);
            uint4 w;
            encode_record<HOT, HOT>(t, __ldcs(form + j), a, __ldcs(ctrl + j), &w.x, &w.y, &w.z, &w.w);
            __stcs(words + j, w);
        }
        return;
    }
    for (uint64_t i = tid; i < n; i += 2 * step) {
        const uint64_t j = i + step;
        const bool two = j < n;
        uint32_t a[8], b[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] = __ldcs(slots + (uint64_t)k * slot_stride + i);
        const uint32_t fa = __ldcs(form + i), ca = __ldcs(ctrl + i);
        uint32_t fb = FORM_NONE, cb = 0;
        if (two) {
#pragma unroll
            for (int k = 0; k < 8; ++k) b[k] = __ldcs(slots + (uint64_t)k * slot_stride + j);
            fb = __ldcs(form + j); cb = __ldcs(ctrl + j);
        }
        uint4 w;
        encode_record<HOT, HOT>(t, fa, a, ca, &w.x, &w.y, &w.z, &w.w);
        __stcs(words + i, w);
        if (two) {
            encode_record<HOT, HOT>(t, fb, b, cb, &w.x, &w.y, &w.z, &w.w);
            __stcs(words + j, w);
        }
    }
}

template <class HOT, bool WIDE, bool COUNT>
__global__ void __launch_bounds__(std::is_same<HOT, HotGlobal>::value ? kBlock : kBlockShared, 1)
roundtrip_kernel(FlatView tg, const uint4* __restrict__ words, uint64_t n, uint8_t* __restrict__ status,
                 unsigned long long* counters) {
    stage_table<HOT>(tg, 0, tg.at.hot_words);
    const FlatView& t = tg;
    uint32_t n_exact = 0, n_rejected = 0;
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    // The next word of a thread is loaded before the current one is checked.
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (first < n) w = __ldcs(words + first);
    for (uint64_t i = first; i < n; i += step) {
        uint4 next = w;
        if (n - i > step) next = __ldcs(words + (i + step));
        const uint32_t st = roundtrip_word<HOT, WIDE>(t, w.x, w.y, w.z, w.w);
        __stcs(status + i, (uint8_t)st);
        if (COUNT) { n_exact += st == RT_EXACT; n_rejected += st == RT_REJECTED; }
        w = next;
    }
    if (COUNT) {
        const uint32_t seen = first < n ? (uint32_t)((n - first + step - 1) / step) : 0u;
        const uint32_t tally[3] = {n_exact, seen - n_exact - n_rejected, n_rejected};
        const int which[3] = {CNT_EXACT, CNT_MISMATCH, CNT_REJECTED};
        block_tally(tally, which, counters);
    }
}

// Per-kernel metadata reduction: every word of every kernel in one launch.  word_start
// (n_kernels + 1 entries) maps a word index to its kernel; results are combined per warp
// when the whole warp sits in one kernel, else per lane.
template <class HOT>
__global__ void __launch_bounds__(std::is_same<HOT, HotGlobal>::value ? kBlock : kBlockShared)
meta_kernel(FlatView tg, const uint4* __restrict__ words, uint64_t n, const uint64_t* __restrict__ word_start,
            uint32_t n_kernels, uint32_t* __restrict__ max_reg, uint32_t* __restrict__ barriers,
            uint8_t* __restrict__ exit_flag) {
    stage_table<HOT>(tg, 0, tg.at.hot_words);
    const FlatView& t = tg;
    const uint64_t step = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t base = (uint64_t)blockIdx.x * blockDim.x; base < n; base += step) {
        const uint64_t i = base + threadIdx.x;
        const bool live = i < n;
        uint32_t mr = 0, bm = 0, ex = 0, k = 0;
        if (live) {
            const uint4 w = __ldcs(words + i);
            word_meta<HOT>(t, w.x, w.y, w.z, &mr, &bm, &ex);
            uint32_t lo = 0, hi = n_kernels;   // last kernel whose first word is <= i
            while (hi - lo > 1) {
                const uint32_t mid = (lo + hi) >> 1;
                if (__ldg(word_start + mid) <= i) lo = mid; else hi = mid;
            }
            k = lo;
            exit_flag[i] = (uint8_t)ex;
        }
        const uint32_t k0 = __shfl_sync(0xFFFFFFFFu, k, 0);
        if (__all_sync(0xFFFFFFFFu, live && k == k0)) {
            mr = __reduce_max_sync(0xFFFFFFFFu, mr);
            bm = __reduce_or_sync(0xFFFFFFFFu, bm);
            if ((threadIdx.x & 31) == 0) {
                if (mr) atomicMax(max_reg + k0, mr);
                if (bm) atomicOr(barriers + k0, bm);
            }
        } else if (live) {
            if (mr) atomicMax(max_reg + k, mr);
            if (bm) atomicOr(barriers + k, bm);
        }
    }
}

__global__ void __launch_bounds__(kBlock)
synth_kernel(FlatView t, SynthView g, uint64_t first, uint64_t n, uint4* __restrict__ words,
             uint16_t* __restrict__ form, uint32_t* __restrict__ slots, uint64_t slot_stride,
             uint32_t* __restrict__ ctrl) {
    const uint64_t step = (uint64_t)gridDim.x * kBlock;
    for (uint64_t i = (uint64_t)blockIdx.x * kBlock + threadIdx.x; i < n; i += step) {
        uint32_t f = FORM_NONE, c = 0, s[8] = {0, 0, 0, 0, 0, 0, 0, 0}, w[4];
        if (synth_record(t, g, first + i, &f, s, &c, w)) encode_record<HotGlobal, HotGlobal>(t, f, s, c, &w[0], &w[1], &w[2], &w[3]);
        else c = ctrl_from_raw(w[0], w[3]);
        if (words) words[i] = make_uint4(w[0], w[1], w[2], w[3]);
        if (form) form[i] = (uint16_t)f;
        if (ctrl) ctrl[i] = c;
        if (slots)
            for (int k = 0; k < 8; ++k) slots[(uint64_t)k * slot_stride + i] = s[k];
    }
}

// ---- scratch of the allocation-free entry point ----------------------------------------------
//
// cubit_decode_batch_static stages one batch through this array instead of memory from
// cudaMalloc: the words, the three record planes the kernel writes, and the launch counters.
// It is part of the library image, so every GPU that loads the library carries it
// (about 3.4 MiB) until the process exits.  In host code the name below is only a handle for
// cudaGetSymbolAddress; the kernel is given the device address obtained from it.
constexpr uint64_t kStaticMaxWords = CUBIT_STATIC_MAX_WORDS;
constexpr uint64_t kStaticFormOff = kStaticMaxWords * 16;
constexpr uint64_t kStaticSlotsOff = kStaticFormOff + kStaticMaxWords * 2;
constexpr uint64_t kStaticCtrlOff = kStaticSlotsOff + kStaticMaxWords * 32;
constexpr uint64_t kStaticCountersOff = kStaticCtrlOff + kStaticMaxWords * 4;
constexpr uint64_t kStaticBytes = kStaticCountersOff + 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];
// One array per GPU whatever the number of contexts: its users are serialised per device ordinal,
// and its device address there is looked up once.
constexpr int kMaxStaticDevices = 64;
std::mutex g_static_mu[kMaxStaticDevices];
unsigned char* g_static_addr[kMaxStaticDevices] = {nullptr};

// ---- context -----------------------------------------------------------------------------

thread_local std::string g_create_error;

struct DeviceState {
    int device = -1;
    int sm_count = 0;
    bool wide_leaves = false; // the table has a leaf of more than 16 classes: kernels with the wide-leaf path
    bool wide_index = false;  // CUBIT_WIDE_INDEX=1: 64-bit word indices at every batch size (otherwise only above 2^31 words)
    bool shared_ok = false;   // the hot part of the table fits the opt-in shared memory of this device
    bool rt_shared_ok = false;   // so do the roundtrip kernel's two ranges (selection tables + roundtrip constants)
    uint32_t rt_bytes = 0;
    uint32_t hot_bytes = 0;   // decode window of the table
    uint32_t enc_bytes = 0;   // encode window
    FlatView view{};
    std::vector<void*> table_allocs;
    unsigned long long* counters = nullptr;   // kCounterSlots x CNT_WORDS
    std::vector<int> free_counter_slots;
    std::mutex mu;
    // Grow-only staging for the host-memory paths.
    void* stage = nullptr;
    uint64_t stage_bytes = 0;
    cudaStream_t stream = nullptr, stream2 = nullptr;
    cudaEvent_t event = nullptr;
    std::mutex stage_mu;
    // Stream generator tables, one per (mix, seed).
    std::map<std::pair<uint32_t, uint64_t>, SynthView> synth;
};
constexpr int kCounterSlots = 64;

}  // namespace

struct cubit_ctx {
    IsaTable table;
    FlatTable flat;
    std::vector<std::unique_ptr<DeviceState>> devs;
    std::map<std::pair<std::string, std::string>, uint32_t> by_name;
    std::vector<std::vector<cubit_field_info>> field_infos;
    std::mutex err_mu;
    std::map<std::thread::id, std::string> errors;
    std::mutex synth_mu;
    // Host-side fault injection for tests (read from the environment when the context is made):
    // CUBIT_TEST_FAIL_SLOT=k makes the worker of device slot k report a failure instead of running,
    // CUBIT_TEST_FAIL_ALLOC=1 makes every growth of a staging buffer fail.  Nothing on a GPU is faulted.
    int test_fail_slot = -1;
    bool test_fail_alloc = false;
    std::unique_ptr<TextEncoder> text;   // built with the context; reads `table`
    std::vector<VariantPrintCache> print_cache;   // per variant, for the printer
};

struct cubit_elf {
    const uint8_t* bytes;
    uint64_t len;
    std::vector<TextSection> text;
};

namespace {

int fail(const cubit_ctx* ctx, int code, const std::string& msg) {
    if (ctx) {
        cubit_ctx* c = const_cast<cubit_ctx*>(ctx);
        std::lock_guard<std::mutex> g(c->err_mu);
        c->errors[std::this_thread::get_id()] = msg;
    } else {
        g_create_error = msg;
    }
    return code;
}

// What an exported function returns when an exception reaches its outermost handler: nothing
// may propagate into the caller's C frames.
int translate_exception(const cubit_ctx* ctx) noexcept {
    try {
        try {
            throw;
        } catch (const TextError& e) {
            return fail(ctx, CUBIT_ERR_TEXT, e.what());
        } catch (const std::bad_alloc&) {
            return fail(ctx, CUBIT_ERR_NOMEM, "out of host memory");
        } catch (const std::exception& e) {
            return fail(ctx, CUBIT_ERR_INVALID, e.what());
        } catch (...) {
            return fail(ctx, CUBIT_ERR_INVALID, "unknown failure");
        }
    } catch (...) {   // recording the message failed as well
        return CUBIT_ERR_NOMEM;
    }
}

#define CU_TRY(ctx, call)                                                                             \
    do {                                                                                              \
        cudaError_t e_ = (call);                                                                      \
        if (e_ != cudaSuccess)                                                                        \
            return fail(ctx, CUBIT_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_));     \
    } while (0)

// The same for calls that follow asynchronous work on `stream`: what was queued is waited for
// before the error is returned, so that nothing still writes into the caller's buffers, local
// arrays or the staging area when the staging lock is dropped.
#define CU_TRY_DRAIN(ctx, stream, call)                                                               \
    do {                                                                                              \
        cudaError_t e_ = (call);                                                                      \
        if (e_ != cudaSuccess) {                                                                      \
            cudaStreamSynchronize(stream);                                                            \
            cudaGetLastError();                                                                       \
            return fail(ctx, CUBIT_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_));     \
        }                                                                                             \
    } while (0)

// Frees what one device of a context holds; the device is made current first.
void release_device(DeviceState* d) {
    if (cudaSetDevice(d->device) != cudaSuccess) { cudaGetLastError(); return; }
    cudaDeviceSynchronize();
    for (void* p : d->table_allocs) cudaFree(p);
    d->table_allocs.clear();
    if (d->counters) cudaFree(d->counters);
    if (d->stage) cudaFree(d->stage);
    if (d->stream) cudaStreamDestroy(d->stream);
    if (d->stream2) cudaStreamDestroy(d->stream2);
    if (d->event) cudaEventDestroy(d->event);
    d->counters = nullptr; d->stage = nullptr; d->stream = d->stream2 = nullptr; d->event = nullptr;
}

std::string bundled_table_path() {
    Dl_info info;
    if (dladdr((void*)&bundled_table_path, &info) && info.dli_fname) {
        std::string p(info.dli_fname);
        size_t slash = p.rfind('/');
        std::string dir = slash == std::string::npos ? "." : p.substr(0, slash);
        return dir + "/../tables/sm120.json";
    }
    return "tables/sm120.json";
}

template <typename T>
int upload(cubit_ctx* ctx, DeviceState* d, const std::vector<T>& host, const T** out) {
    void* p = nullptr;
    const size_t bytes = std::max<size_t>(host.size() * sizeof(T), 16);
    CU_TRY(ctx, cudaMalloc(&p, bytes));
    d->table_allocs.push_back(p);
    if (!host.empty()) CU_TRY(ctx, cudaMemcpy(p, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice));
    *out = (const T*)p;
    return CUBIT_OK;
}

// Uploads the table to one device and creates its streams and counters.  Failures report
// through the thread-local message, as the context does not exist yet for the caller.
int init_device(const FlatTable& ft, DeviceState* d) {
    cubit_ctx* c = nullptr;
    CU_TRY(c, cudaSetDevice(d->device));
    CU_TRY(c, cudaDeviceGetAttribute(&d->sm_count, cudaDevAttrMultiProcessorCount, d->device));
    const uint32_t* blob = nullptr;
    const int rc = upload(c, d, ft.blob, &blob);
    if (rc) return rc;
    d->view.cold = blob; d->view.at = ft.at;
    d->hot_bytes = ft.at.hot_words * 4;
    d->wide_leaves = ft.max_leaf_classes > 16;
    {
        const char* wide = getenv("CUBIT_WIDE_INDEX");
        d->wide_index = wide && wide[0] == '1';
    }
    d->enc_bytes = (ft.at.enc_end - ft.at.enc) * 4;
    int optin = 0;
    CU_TRY(c, cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, d->device));
    d->shared_ok = (int)d->hot_bytes + 1024 <= optin && (int)d->enc_bytes + 1024 <= optin;
    if (d->shared_ok) {
        const int hot = (int)d->hot_bytes;
#define CB_DECODE_SMEM(IDX, WIDE, COUNT) \
        CU_TRY(c, cudaFuncSetAttribute(decode_kernel<HotShared, IDX, WIDE, COUNT>, cudaFuncAttributeMaxDynamicSharedMemorySize, hot))
        CB_DECODE_SMEM(uint32_t, true, true); CB_DECODE_SMEM(uint32_t, true, false);
        CB_DECODE_SMEM(uint64_t, true, true); CB_DECODE_SMEM(uint64_t, true, false);
        CB_DECODE_SMEM(uint32_t, false, true); CB_DECODE_SMEM(uint32_t, false, false);
        CB_DECODE_SMEM(uint64_t, false, true); CB_DECODE_SMEM(uint64_t, false, false);
#undef CB_DECODE_SMEM
        CU_TRY(c, cudaFuncSetAttribute(encode_kernel<HotSharedEnc>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d->enc_bytes));
        CU_TRY(c, cudaFuncSetAttribute(roundtrip_kernel<HotShared, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, hot));
        CU_TRY(c, cudaFuncSetAttribute(roundtrip_kernel<HotShared, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, hot));
        CU_TRY(c, cudaFuncSetAttribute(roundtrip_kernel<HotShared, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, hot));
        CU_TRY(c, cudaFuncSetAttribute(roundtrip_kernel<HotShared, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, hot));
        CU_TRY(c, cudaFuncSetAttribute(meta_kernel<HotShared>, cudaFuncAttributeMaxDynamicSharedMemorySize, hot));
    }
    d->rt_bytes = (ft.at.sel_words + (ft.at.total_words - ft.at.rt[0])) * 4;
    d->rt_shared_ok = d->shared_ok && (int)d->rt_bytes + 1024 <= optin;
    if (d->rt_shared_ok) {
        CU_TRY(c, cudaFuncSetAttribute(roundtrip_kernel<HotSharedRT, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d->rt_bytes));
        CU_TRY(c, cudaFuncSetAttribute(roundtrip_kernel<HotSharedRT, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d->rt_bytes));
        CU_TRY(c, cudaFuncSetAttribute(roundtrip_kernel<HotSharedRT, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d->rt_bytes));
        CU_TRY(c, cudaFuncSetAttribute(roundtrip_kernel<HotSharedRT, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d->rt_bytes));
    }
    CU_TRY(c, cudaMalloc((void**)&d->counters, sizeof(unsigned long long) * CNT_WORDS * kCounterSlots));
    for (int s = 0; s < kCounterSlots; ++s) d->free_counter_slots.push_back(s);
    CU_TRY(c, cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
    CU_TRY(c, cudaStreamCreateWithFlags(&d->stream2, cudaStreamNonBlocking));
    CU_TRY(c, cudaEventCreateWithFlags(&d->event, cudaEventDisableTiming));
    return CUBIT_OK;
}

int grid_for(const DeviceState* d, uint64_t n) {
    const uint64_t blocks = (n + kBlock - 1) / kBlock;
    const uint64_t cap = (uint64_t)d->sm_count * 8;   // whole waves of resident blocks
    return (int)std::max<uint64_t>(1, std::min(blocks, cap));
}

// Large batches run on persistent CTAs with the table in shared memory.
bool use_shared(const DeviceState* d, uint64_t n) { return d->shared_ok && n >= kSharedMinWords; }
int grid_shared(const DeviceState* d, uint64_t n) {
    return (int)std::max<uint64_t>(1, std::min<uint64_t>((n + kBlockShared - 1) / kBlockShared, (uint64_t)d->sm_count));
}

void launch_decode(const DeviceState* d, cudaStream_t s, const uint4* words, uint64_t n, uint16_t* form, uint32_t* slots,
                   uint64_t stride, uint32_t* ctrl, unsigned long long* dc) {
    // 32-bit word indices while index + grid size cannot wrap; kernels without the wide-leaf path when the
    // table has no such leaf.
    const bool narrow = n < (1ull << 31) && !d->wide_index;
    const bool staged = use_shared(d, n);
    const int grid = staged ? grid_shared(d, n) : grid_for(d, n), block = staged ? kBlockShared : kBlock;
    const size_t smem = staged ? d->hot_bytes : 0;
#define CB_LAUNCH_DECODE(HOT, IDX, WIDE)                                                                             \
    do {                                                                                                             \
        if (dc) decode_kernel<HOT, IDX, WIDE, true><<<grid, block, smem, s>>>(d->view, words, n, form, slots, stride, ctrl, dc); \
        else decode_kernel<HOT, IDX, WIDE, false><<<grid, block, smem, s>>>(d->view, words, n, form, slots, stride, ctrl, dc);  \
    } while (0)
    if (staged) {
        if (d->wide_leaves) { if (narrow) CB_LAUNCH_DECODE(HotShared, uint32_t, true); else CB_LAUNCH_DECODE(HotShared, uint64_t, true); }
        else { if (narrow) CB_LAUNCH_DECODE(HotShared, uint32_t, false); else CB_LAUNCH_DECODE(HotShared, uint64_t, false); }
    } else {
        if (d->wide_leaves) { if (narrow) CB_LAUNCH_DECODE(HotGlobal, uint32_t, true); else CB_LAUNCH_DECODE(HotGlobal, uint64_t, true); }
        else { if (narrow) CB_LAUNCH_DECODE(HotGlobal, uint32_t, false); else CB_LAUNCH_DECODE(HotGlobal, uint64_t, false); }
    }
#undef CB_LAUNCH_DECODE
}
void launch_encode(const DeviceState* d, cudaStream_t s, const uint16_t* form, const uint32_t* slots, uint64_t stride,
                   const uint32_t* ctrl, uint64_t n, uint4* words) {
    // 64-bit loads of two neighbouring records need every plane 8-byte aligned.
    const int paired = (stride % 2 == 0) && ((uintptr_t)slots % 8 == 0) && ((uintptr_t)ctrl % 8 == 0) &&
                       ((uintptr_t)form % 4 == 0);
    if (use_shared(d, n))
        encode_kernel<HotSharedEnc><<<grid_shared(d, n), kBlockShared, d->enc_bytes, s>>>(d->view, form, slots, stride, ctrl, n, words, paired);
    else
        encode_kernel<HotGlobal><<<grid_for(d, n), kBlock, 0, s>>>(d->view, form, slots, stride, ctrl, n, words, paired);
}
void launch_roundtrip(const DeviceState* d, cudaStream_t s, const uint4* words, uint64_t n, uint8_t* status,
                      unsigned long long* dc) {
#define CB_LAUNCH_RT(HOT, grid, block, smem)                                                          \
    do {                                                                                              \
        if (d->wide_leaves) {                                                                         \
            if (dc) roundtrip_kernel<HOT, true, true><<<grid, block, smem, s>>>(d->view, words, n, status, dc);   \
            else roundtrip_kernel<HOT, true, false><<<grid, block, smem, s>>>(d->view, words, n, status, dc);     \
        } else {                                                                                      \
            if (dc) roundtrip_kernel<HOT, false, true><<<grid, block, smem, s>>>(d->view, words, n, status, dc);  \
            else roundtrip_kernel<HOT, false, false><<<grid, block, smem, s>>>(d->view, words, n, status, dc);    \
        }                                                                                             \
    } while (0)
    if (use_shared(d, n) && d->rt_shared_ok) CB_LAUNCH_RT(HotSharedRT, grid_shared(d, n), kBlockShared, d->rt_bytes);
    else if (use_shared(d, n)) CB_LAUNCH_RT(HotShared, grid_shared(d, n), kBlockShared, d->hot_bytes);
    else CB_LAUNCH_RT(HotGlobal, grid_for(d, n), kBlock, 0);
#undef CB_LAUNCH_RT
}

DeviceState* device_of_pointer(cubit_ctx* ctx, const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (a.type != cudaMemoryTypeDevice && a.type != cudaMemoryTypeManaged) return nullptr;
    for (auto& d : ctx->devs)
        if (d->device == a.device) return d.get();
    return nullptr;
}

int take_counter_slot(DeviceState* d) {
    std::lock_guard<std::mutex> g(d->mu);
    if (d->free_counter_slots.empty()) return -1;
    int s = d->free_counter_slots.back();
    d->free_counter_slots.pop_back();
    return s;
}
void give_counter_slot(DeviceState* d, int s) {
    std::lock_guard<std::mutex> g(d->mu);
    d->free_counter_slots.push_back(s);
}

void add_counts(cubit_counts* out, const unsigned long long* c) {
    out->n_decoded += c[CNT_DECODED]; out->n_rejected += c[CNT_REJECTED]; out->n_tie += c[CNT_TIE];
    out->n_exact += c[CNT_EXACT]; out->n_mismatch += c[CNT_MISMATCH];
}

// Runs `launch(counters)` on `stream` of device d; when counts are wanted, zeroes a counter
// slot first and reads it back (which waits for the stream).
template <typename Launch>
int run_counted(cubit_ctx* ctx, DeviceState* d, cudaStream_t stream, cubit_counts* counts, Launch launch) {
    if (!counts) {
        launch((unsigned long long*)nullptr);
        CU_TRY(ctx, cudaGetLastError());
        return CUBIT_OK;
    }
    const int slot = take_counter_slot(d);
    if (slot < 0) return fail(ctx, CUBIT_ERR_NOMEM, "too many counted calls in flight on one device");
    unsigned long long* dc = d->counters + (size_t)slot * CNT_WORDS;
    unsigned long long host[CNT_WORDS];
    cudaError_t e = cudaMemsetAsync(dc, 0, sizeof host, stream);
    if (e == cudaSuccess) { launch(dc); e = cudaGetLastError(); }
    if (e == cudaSuccess) e = cudaMemcpyAsync(host, dc, sizeof host, cudaMemcpyDeviceToHost, stream);
    // The slot goes back only when nothing queued above can still write to it or to `host`.
    const cudaError_t waited = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) e = waited;
    give_counter_slot(d, slot);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, CUBIT_ERR_CUDA, std::string("counted launch: ") + cudaGetErrorString(e));
    }
    add_counts(counts, host);
    return CUBIT_OK;
}

int ensure_stage(cubit_ctx* ctx, DeviceState* d, uint64_t bytes) {
    if (d->stage_bytes >= bytes) return CUBIT_OK;
    if (ctx->test_fail_alloc) return fail(ctx, CUBIT_ERR_NOMEM, "staging buffer allocation failed (injected by CUBIT_TEST_FAIL_ALLOC)");
    if (d->stage) { CU_TRY(ctx, cudaFree(d->stage)); d->stage = nullptr; d->stage_bytes = 0; }
    CU_TRY(ctx, cudaMalloc(&d->stage, bytes));
    d->stage_bytes = bytes;
    return CUBIT_OK;
}

// Contiguous range of device k out of g for n items.
void shard_range(uint64_t n, size_t g, size_t k, uint64_t* begin, uint64_t* end) {
    *begin = n / g * k + std::min<uint64_t>(k, n % g);
    *end = *begin + n / g + (k < n % g ? 1 : 0);
}

constexpr uint64_t kChunkWords = 1ull << 22;   // host paths stream the batch in 4 Mi-word chunks

uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// One chunk of a host batch on its way through the device: the stream it is queued on, its half
// of the staging area, the first item and the number of items, and the counter slot of the call.
struct ChunkIO {
    cudaStream_t stream;
    uint8_t* stage;
    uint64_t at, items;
    unsigned long long* counters;
};

// Streams items [begin, end) of a host batch through one device.  The range is cut into chunks
// that alternate between two halves of the staging area and two streams, so the copy-in of one
// chunk, the kernel of another and the copy-out of a third overlap (the PCIe link is full
// duplex); with pinned host buffers every copy is asynchronous.  `body` queues the copies and
// the launch of one chunk on the chunk's stream and returns the first CUDA error it met.
// The caller holds the device's staging lock and has made the device current.  Whatever fails,
// nothing is left running on either stream when this returns.
template <typename Body>
int pipeline_host_range(cubit_ctx* ctx, DeviceState* d, uint64_t begin, uint64_t end, uint64_t chunk, uint64_t half,
                        cubit_counts* counts, const char* what, Body body) {
    const bool two = end - begin > chunk;
    int rc = ensure_stage(ctx, d, two ? 2 * half : half);
    if (rc) return rc;
    int slot = -1;
    unsigned long long* dc = nullptr;
    if (counts) {
        slot = take_counter_slot(d);
        if (slot < 0) return fail(ctx, CUBIT_ERR_NOMEM, "too many counted calls in flight on one device");
        dc = d->counters + (size_t)slot * CNT_WORDS;
    }
    cudaStream_t streams[2] = {d->stream, d->stream2};
    cudaError_t e = cudaSuccess;
    if (dc) {
        e = cudaMemsetAsync(dc, 0, sizeof(unsigned long long) * CNT_WORDS, streams[0]);
        if (e == cudaSuccess) e = cudaEventRecord(d->event, streams[0]);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(streams[1], d->event, 0);
    }
    uint64_t k = 0;
    for (uint64_t at = begin; at < end && e == cudaSuccess; at += chunk, ++k)
        e = body(ChunkIO{streams[k & 1], (uint8_t*)d->stage + (k & 1) * half, at, std::min(chunk, end - at), dc});
    unsigned long long host[CNT_WORDS] = {0, 0, 0, 0, 0};
    if (e == cudaSuccess) e = cudaStreamSynchronize(streams[1]);
    if (e == cudaSuccess && dc) e = cudaMemcpyAsync(host, dc, sizeof host, cudaMemcpyDeviceToHost, streams[0]);
    if (e == cudaSuccess) e = cudaStreamSynchronize(streams[0]);
    if (e != cudaSuccess) {   // nothing may still be using the staging area, the caller's buffers or the counter slot
        cudaStreamSynchronize(streams[0]);
        cudaStreamSynchronize(streams[1]);
        cudaGetLastError();
    }
    if (slot >= 0) give_counter_slot(d, slot);
    if (e != cudaSuccess) return fail(ctx, CUBIT_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    if (counts) add_counts(counts, host);
    return CUBIT_OK;
}

// Staging layout of one chunk of records: words, then the form, slot and ctrl planes.
struct RecordStage {
    uint64_t chunk, o_form, o_slots, o_ctrl, half;
    explicit RecordStage(uint64_t items) {
        chunk = std::min<uint64_t>(kChunkWords, std::max<uint64_t>(items, 1));
        o_form = align_up(chunk * 16, 256);
        o_slots = o_form + align_up(chunk * 2, 256);
        o_ctrl = o_slots + chunk * 32;
        half = align_up(o_ctrl + chunk * 4, 256);
    }
};

// Queues the copy of one chunk's records from the staging area to host planes that are
// `host_stride` records apart, record `at` of the call landing at `host_at`.
cudaError_t records_to_host(const RecordStage& L, const ChunkIO& io, uint64_t host_at, uint64_t host_stride, uint16_t* form,
                            uint32_t* slots, uint32_t* ctrl) {
    cudaError_t e = cudaSuccess;
    if (form) e = cudaMemcpyAsync(form + host_at, io.stage + L.o_form, io.items * 2, cudaMemcpyDeviceToHost, io.stream);
    for (int p = 0; p < 8 && e == cudaSuccess && slots; ++p)
        e = cudaMemcpyAsync(slots + (uint64_t)p * host_stride + host_at, io.stage + L.o_slots + (uint64_t)p * L.chunk * 4,
                            io.items * 4, cudaMemcpyDeviceToHost, io.stream);
    if (e == cudaSuccess && ctrl) e = cudaMemcpyAsync(ctrl + host_at, io.stage + L.o_ctrl, io.items * 4, cudaMemcpyDeviceToHost, io.stream);
    return e;
}

// Host-memory decode of words [begin, end) on one device.
int decode_host_range(cubit_ctx* ctx, DeviceState* d, const uint8_t* words, uint64_t n_total, uint64_t begin,
                      uint64_t end, uint16_t* form, uint32_t* slots, uint32_t* ctrl, cubit_counts* counts) {
    std::lock_guard<std::mutex> g(d->stage_mu);
    CU_TRY(ctx, cudaSetDevice(d->device));
    const RecordStage L(end - begin);
    return pipeline_host_range(ctx, d, begin, end, L.chunk, L.half, counts, "host decode", [&](const ChunkIO& io) {
        cudaError_t e = cudaMemcpyAsync(io.stage, words + io.at * 16, io.items * 16, cudaMemcpyHostToDevice, io.stream);
        if (e != cudaSuccess) return e;
        launch_decode(d, io.stream, (const uint4*)io.stage, io.items, (uint16_t*)(io.stage + L.o_form),
                      (uint32_t*)(io.stage + L.o_slots), L.chunk, (uint32_t*)(io.stage + L.o_ctrl), io.counters);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = records_to_host(L, io, io.at, n_total, form, slots, ctrl);
        return e;
    });
}

int encode_host_range(cubit_ctx* ctx, DeviceState* d, const uint16_t* form, const uint32_t* slots, const uint32_t* ctrl,
                      uint64_t n_total, uint64_t begin, uint64_t end, uint8_t* words) {
    std::lock_guard<std::mutex> g(d->stage_mu);
    CU_TRY(ctx, cudaSetDevice(d->device));
    const RecordStage L(end - begin);
    return pipeline_host_range(ctx, d, begin, end, L.chunk, L.half, nullptr, "host encode", [&](const ChunkIO& io) {
        cudaError_t e = cudaMemcpyAsync(io.stage + L.o_form, form + io.at, io.items * 2, cudaMemcpyHostToDevice, io.stream);
        for (int k = 0; k < 8 && e == cudaSuccess; ++k)
            e = cudaMemcpyAsync(io.stage + L.o_slots + (uint64_t)k * L.chunk * 4, slots + (uint64_t)k * n_total + io.at,
                                io.items * 4, cudaMemcpyHostToDevice, io.stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(io.stage + L.o_ctrl, ctrl + io.at, io.items * 4, cudaMemcpyHostToDevice, io.stream);
        if (e != cudaSuccess) return e;
        launch_encode(d, io.stream, (const uint16_t*)(io.stage + L.o_form), (const uint32_t*)(io.stage + L.o_slots), L.chunk,
                      (const uint32_t*)(io.stage + L.o_ctrl), io.items, (uint4*)io.stage);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpyAsync(words + io.at * 16, io.stage, io.items * 16, cudaMemcpyDeviceToHost, io.stream);
        return e;
    });
}

int roundtrip_host_range(cubit_ctx* ctx, DeviceState* d, const uint8_t* words, uint64_t begin, uint64_t end,
                         uint8_t* status, cubit_counts* counts) {
    std::lock_guard<std::mutex> g(d->stage_mu);
    CU_TRY(ctx, cudaSetDevice(d->device));
    const uint64_t chunk = std::min<uint64_t>(kChunkWords, std::max<uint64_t>(end - begin, 1));
    const uint64_t o_status = align_up(chunk * 16, 256), half = align_up(o_status + chunk, 256);
    return pipeline_host_range(ctx, d, begin, end, chunk, half, counts, "host roundtrip", [&](const ChunkIO& io) {
        cudaError_t e = cudaMemcpyAsync(io.stage, words + io.at * 16, io.items * 16, cudaMemcpyHostToDevice, io.stream);
        if (e != cudaSuccess) return e;
        launch_roundtrip(d, io.stream, (const uint4*)io.stage, io.items, io.stage + o_status, io.counters);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpyAsync(status + io.at, io.stage + o_status, io.items, cudaMemcpyDeviceToHost, io.stream);
        return e;
    });
}

// Runs fn(device index) for every device of the context on its own host thread and merges
// the per-device counts and status codes.
template <typename Fn>
int for_each_device(cubit_ctx* ctx, cubit_counts* counts, Fn fn) {
    const size_t g = ctx->devs.size();
    std::vector<int> rcs(g, CUBIT_OK);
    std::vector<cubit_counts> partial(g);
    std::vector<std::string> messages(g);
    memset(partial.data(), 0, g * sizeof(cubit_counts));
    auto body = [&](size_t k) {
        if (ctx->test_fail_slot == (int)k)
            rcs[k] = fail(ctx, CUBIT_ERR_CUDA, "device slot " + std::to_string(k) + " failed (injected by CUBIT_TEST_FAIL_SLOT)");
        else
            rcs[k] = fn(k, counts ? &partial[k] : nullptr);
        if (rcs[k]) messages[k] = cubit_last_error(ctx);
        if (g > 1) {   // a worker thread ends here: its message slot goes with it
            std::lock_guard<std::mutex> lock(ctx->err_mu);
            ctx->errors.erase(std::this_thread::get_id());
        }
    };
    if (g == 1) {
        body(0);
    } else {
        std::vector<std::thread> th;
        for (size_t k = 0; k < g; ++k) th.emplace_back(body, k);
        for (auto& t : th) t.join();
    }
    for (size_t k = 0; k < g; ++k)
        if (rcs[k]) return fail(ctx, rcs[k], messages[k]);
    if (counts)
        for (size_t k = 0; k < g; ++k) {
            counts->n_decoded += partial[k].n_decoded; counts->n_rejected += partial[k].n_rejected;
            counts->n_tie += partial[k].n_tie; counts->n_exact += partial[k].n_exact;
            counts->n_mismatch += partial[k].n_mismatch;
        }
    return CUBIT_OK;
}

int get_synth_view(cubit_ctx* ctx, DeviceState* d, uint32_t mix, uint64_t seed, uint32_t noise_ppm, SynthView* out) {
    std::lock_guard<std::mutex> g(ctx->synth_mu);
    const uint64_t table_seed = mix == MIX_ZIPF ? seed : 0;   // only the Zipf permutation depends on the seed
    auto key = std::make_pair(mix, table_seed);
    auto it = d->synth.find(key);
    if (it == d->synth.end()) {
        SynthTables st;
        try {
            st = build_synth_tables(ctx->table, mix, seed);
        } catch (const std::exception& e) {
            return fail(ctx, CUBIT_ERR_INVALID, e.what());
        }
        CU_TRY(ctx, cudaSetDevice(d->device));
        SynthView v{};
        int rc = upload(ctx, d, st.cdf, &v.cdf);
        if (!rc) rc = upload(ctx, d, st.rank_first, &v.rank_first);
        if (!rc) rc = upload(ctx, d, st.rank_count, &v.rank_count);
        if (rc) return rc;
        v.n_ranks = (uint32_t)st.cdf.size();
        it = d->synth.emplace(key, v).first;
    }
    *out = it->second;
    out->seed = seed;
    out->noise_ppm = noise_ppm;
    return CUBIT_OK;
}

}  // namespace

// ---- exported: context ------------------------------------------------------------------------

extern "C" int cubit_ctx_create(const char* table_path, const int* devices, int n_devices, cubit_ctx** out) try {
    if (!out || n_devices < 0 || (n_devices > 0 && !devices)) return fail(nullptr, CUBIT_ERR_INVALID, "bad argument");
    *out = nullptr;
    std::unique_ptr<cubit_ctx> ctx(new cubit_ctx);
    std::string path;
    const char* env = getenv("CUBIT_TABLE");
    if (env && *env) path = env;
    else if (table_path && *table_path) path = table_path;
    else path = bundled_table_path();
    try {
        ctx->table = IsaTable::from_file(path);
        ctx->flat = FlatTable::compile(ctx->table);
    } catch (const std::exception& e) {
        return fail(nullptr, CUBIT_ERR_TABLE, std::string("table ") + path + ": " + e.what());
    }
    const FlatTable& ft = ctx->flat;
    if (const char* slot = getenv("CUBIT_TEST_FAIL_SLOT")) ctx->test_fail_slot = *slot ? atoi(slot) : -1;
    if (const char* alloc = getenv("CUBIT_TEST_FAIL_ALLOC")) ctx->test_fail_alloc = alloc[0] == '1';
    ctx->text.reset(new TextEncoder(ctx->table));
    for (const VariantMeta& m : ft.meta) ctx->print_cache.push_back(make_print_cache(m.key, m.opcode, m.mod_group));
    ctx->field_infos.resize(ft.meta.size());
    for (size_t v = 0; v < ft.meta.size(); ++v) {
        ctx->by_name[{ft.meta[v].key, ft.meta[v].mod_group}] = (uint32_t)v;
        for (const FieldMeta& f : ft.meta[v].fields)
            ctx->field_infos[v].push_back(
                cubit_field_info{f.shift, f.bits, f.token_idx, f.dst_pos, f.stored_bits, f.name.c_str(), f.extraction.c_str()});
    }
    for (int k = 0; k < n_devices; ++k) {
        std::unique_ptr<DeviceState> d(new DeviceState);
        d->device = devices[k];
        const int rc = init_device(ft, d.get());
        if (rc) {   // give back what this and the earlier devices already hold
            release_device(d.get());
            for (auto& made : ctx->devs) release_device(made.get());
            return rc;
        }
        ctx->devs.push_back(std::move(d));
    }
    *out = ctx.release();
    return CUBIT_OK;
} catch (...) {
    return translate_exception(nullptr);
}

extern "C" void cubit_ctx_destroy(cubit_ctx* ctx) {
    if (!ctx) return;
    for (auto& d : ctx->devs) release_device(d.get());
    delete ctx;
}

extern "C" const char* cubit_last_error(const cubit_ctx* ctx) {
    if (!ctx) return g_create_error.c_str();
    cubit_ctx* c = const_cast<cubit_ctx*>(ctx);
    std::lock_guard<std::mutex> g(c->err_mu);
    return c->errors[std::this_thread::get_id()].c_str();
}

extern "C" int cubit_table_info(const cubit_ctx* ctx, uint32_t* n_keys, uint32_t* n_groups) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (n_keys) *n_keys = (uint32_t)ctx->table.num_keys();
    if (n_groups) *n_groups = (uint32_t)ctx->table.num_groups();
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_variant_lookup(const cubit_ctx* ctx, uint32_t variant, cubit_variant_info* out) try {
    if (!ctx || !out) return CUBIT_ERR_INVALID;
    if (variant >= ctx->flat.meta.size()) return fail(ctx, CUBIT_ERR_NOT_FOUND, "variant id out of range");
    const VariantMeta& m = ctx->flat.meta[variant];
    out->key = m.key.c_str(); out->mod_group = m.mod_group.c_str(); out->opcode = m.opcode.c_str();
    out->key_id = m.key_id; out->layout_kind = m.layout_kind; out->synth_mask = m.synth_mask;
    out->ra_tok = m.ra_tok; out->rb_tok = m.rb_tok;
    out->n_fields = (uint32_t)m.fields.size();
    out->fields = ctx->field_infos[variant].data();
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_variant_find(const cubit_ctx* ctx, const char* key, const char* mod_group, uint32_t* variant) try {
    if (!ctx || !key || !mod_group || !variant) return CUBIT_ERR_INVALID;
    auto it = ctx->by_name.find({key, mod_group});
    if (it == ctx->by_name.end()) return fail(ctx, CUBIT_ERR_NOT_FOUND, std::string("no table entry ") + key + "::" + mod_group);
    *variant = it->second;
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_key_name(const cubit_ctx* ctx, uint32_t key_id, const char** name, uint32_t* first_variant,
                              uint32_t* n_variants) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (key_id >= ctx->table.keys.size()) return fail(ctx, CUBIT_ERR_NOT_FOUND, "key id out of range");
    const IsaKey& k = ctx->table.keys[key_id];
    if (name) *name = k.name.c_str();
    if (first_variant) *first_variant = k.first_variant;
    if (n_variants) *n_variants = k.n_variants;
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_host_alloc(cubit_ctx* ctx, uint64_t bytes, void** out) try {
    if (!ctx || !out) return CUBIT_ERR_INVALID;
    if (ctx->devs.empty()) return fail(ctx, CUBIT_ERR_NO_DEVICE, "context has no CUDA device");
    CU_TRY(ctx, cudaSetDevice(ctx->devs[0]->device));
    CU_TRY(ctx, cudaHostAlloc(out, std::max<uint64_t>(bytes, 1), cudaHostAllocPortable));
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_host_free(cubit_ctx* ctx, void* p) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (p) CU_TRY(ctx, cudaFreeHost(p));
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

// ---- exported: batch codec ----------------------------------------------------------------------

extern "C" int cubit_decode_batch(cubit_ctx* ctx, const void* words, uint64_t n, uint16_t* form, uint32_t* slots,
                                  uint32_t* ctrl, cubit_counts* counts, int mem_kind, void* stream) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (counts) memset(counts, 0, sizeof *counts);
    if (ctx->devs.empty()) return fail(ctx, CUBIT_ERR_NO_DEVICE, "decode needs a CUDA device; this context has none");
    if (n == 0) return CUBIT_OK;
    if (!words || !form || !slots || !ctrl) return fail(ctx, CUBIT_ERR_INVALID, "null buffer");
    if (mem_kind == CUBIT_MEM_DEVICE) {
        DeviceState* d = device_of_pointer(ctx, words);
        if (!d) return fail(ctx, CUBIT_ERR_INVALID, "words is not device memory of one of the context's devices");
        if ((uintptr_t)words % 16) return fail(ctx, CUBIT_ERR_INVALID, "device words must be 16-byte aligned");
        CU_TRY(ctx, cudaSetDevice(d->device));
        cudaStream_t s = (cudaStream_t)stream;
        return run_counted(ctx, d, s, counts, [&](unsigned long long* dc) {
            launch_decode(d, s, (const uint4*)words, n, form, slots, n, ctrl, dc);
        });
    }
    if (mem_kind != CUBIT_MEM_HOST) return fail(ctx, CUBIT_ERR_INVALID, "unknown mem_kind");
    const size_t g = ctx->devs.size();
    return for_each_device(ctx, counts, [&](size_t k, cubit_counts* part) {
        uint64_t b, e;
        shard_range(n, g, k, &b, &e);
        if (b == e) return (int)CUBIT_OK;
        return decode_host_range(ctx, ctx->devs[k].get(), (const uint8_t*)words, n, b, e, form, slots, ctrl, part);
    });
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_encode_batch(cubit_ctx* ctx, const uint16_t* form, const uint32_t* slots, const uint32_t* ctrl,
                                  uint64_t n, void* words, int mem_kind, void* stream) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (ctx->devs.empty()) return fail(ctx, CUBIT_ERR_NO_DEVICE, "encode needs a CUDA device; this context has none");
    if (n == 0) return CUBIT_OK;
    if (!words || !form || !slots || !ctrl) return fail(ctx, CUBIT_ERR_INVALID, "null buffer");
    if (mem_kind == CUBIT_MEM_DEVICE) {
        DeviceState* d = device_of_pointer(ctx, words);
        if (!d) return fail(ctx, CUBIT_ERR_INVALID, "words is not device memory of one of the context's devices");
        if ((uintptr_t)words % 16) return fail(ctx, CUBIT_ERR_INVALID, "device words must be 16-byte aligned");
        CU_TRY(ctx, cudaSetDevice(d->device));
        cudaStream_t s = (cudaStream_t)stream;
        launch_encode(d, s, form, slots, n, ctrl, n, (uint4*)words);
        CU_TRY(ctx, cudaGetLastError());
        return CUBIT_OK;
    }
    if (mem_kind != CUBIT_MEM_HOST) return fail(ctx, CUBIT_ERR_INVALID, "unknown mem_kind");
    const size_t g = ctx->devs.size();
    return for_each_device(ctx, nullptr, [&](size_t k, cubit_counts*) {
        uint64_t b, e;
        shard_range(n, g, k, &b, &e);
        if (b == e) return (int)CUBIT_OK;
        return encode_host_range(ctx, ctx->devs[k].get(), form, slots, ctrl, n, b, e, (uint8_t*)words);
    });
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_roundtrip_batch(cubit_ctx* ctx, const void* words, uint64_t n, uint8_t* status,
                                     cubit_counts* counts, int mem_kind, void* stream) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (counts) memset(counts, 0, sizeof *counts);
    if (ctx->devs.empty()) return fail(ctx, CUBIT_ERR_NO_DEVICE, "roundtrip needs a CUDA device; this context has none");
    if (n == 0) return CUBIT_OK;
    if (!words || !status) return fail(ctx, CUBIT_ERR_INVALID, "null buffer");
    if (mem_kind == CUBIT_MEM_DEVICE) {
        DeviceState* d = device_of_pointer(ctx, words);
        if (!d) return fail(ctx, CUBIT_ERR_INVALID, "words is not device memory of one of the context's devices");
        if ((uintptr_t)words % 16) return fail(ctx, CUBIT_ERR_INVALID, "device words must be 16-byte aligned");
        CU_TRY(ctx, cudaSetDevice(d->device));
        cudaStream_t s = (cudaStream_t)stream;
        return run_counted(ctx, d, s, counts, [&](unsigned long long* dc) {
            launch_roundtrip(d, s, (const uint4*)words, n, status, dc);
        });
    }
    if (mem_kind != CUBIT_MEM_HOST) return fail(ctx, CUBIT_ERR_INVALID, "unknown mem_kind");
    const size_t g = ctx->devs.size();
    return for_each_device(ctx, counts, [&](size_t k, cubit_counts* part) {
        uint64_t b, e;
        shard_range(n, g, k, &b, &e);
        if (b == e) return (int)CUBIT_OK;
        return roundtrip_host_range(ctx, ctx->devs[k].get(), (const uint8_t*)words, b, e, status, part);
    });
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_synth_batch(cubit_ctx* ctx, uint32_t mix, uint64_t seed, uint32_t noise_ppm, uint64_t first,
                                 uint64_t n, void* words, uint16_t* form, uint32_t* slots, uint32_t* ctrl, int mem_kind,
                                 void* stream) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (ctx->devs.empty()) return fail(ctx, CUBIT_ERR_NO_DEVICE, "the stream generator needs a CUDA device");
    if (n == 0) return CUBIT_OK;
    if (noise_ppm > 1000000) return fail(ctx, CUBIT_ERR_INVALID, "noise_ppm above one million");
    if (mem_kind == CUBIT_MEM_DEVICE) {
        const void* probe = words ? words : (form ? (const void*)form : (slots ? (const void*)slots : (const void*)ctrl));
        if (!probe) return fail(ctx, CUBIT_ERR_INVALID, "no output buffer");
        DeviceState* d = device_of_pointer(ctx, probe);
        if (!d) return fail(ctx, CUBIT_ERR_INVALID, "output is not device memory of one of the context's devices");
        SynthView g;
        int rc = get_synth_view(ctx, d, mix, seed, noise_ppm, &g);
        if (rc) return rc;
        CU_TRY(ctx, cudaSetDevice(d->device));
        cudaStream_t s = (cudaStream_t)stream;
        synth_kernel<<<grid_for(d, n), kBlock, 0, s>>>(d->view, g, first, n, (uint4*)words, form, slots, n, ctrl);
        CU_TRY(ctx, cudaGetLastError());
        return CUBIT_OK;
    }
    if (mem_kind != CUBIT_MEM_HOST) return fail(ctx, CUBIT_ERR_INVALID, "unknown mem_kind");
    // Host output: generate on the first device in chunks and copy back.
    DeviceState* d = ctx->devs[0].get();
    SynthView g;
    int rc = get_synth_view(ctx, d, mix, seed, noise_ppm, &g);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(d->stage_mu);
    CU_TRY(ctx, cudaSetDevice(d->device));
    const RecordStage L(n);
    return pipeline_host_range(ctx, d, 0, n, L.chunk, L.half, nullptr, "host stream generator", [&](const ChunkIO& io) {
        synth_kernel<<<grid_for(d, io.items), kBlock, 0, io.stream>>>(d->view, g, first + io.at, io.items, (uint4*)io.stage,
                                                                       (uint16_t*)(io.stage + L.o_form), (uint32_t*)(io.stage + L.o_slots),
                                                                       L.chunk, (uint32_t*)(io.stage + L.o_ctrl));
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess && words)
            e = cudaMemcpyAsync((uint8_t*)words + io.at * 16, io.stage, io.items * 16, cudaMemcpyDeviceToHost, io.stream);
        if (e == cudaSuccess) e = records_to_host(L, io, io.at, n, form, slots, ctrl);
        return e;
    });
} catch (...) {
    return translate_exception(ctx);
}

// Host-buffer decode of a small batch that allocates nothing: see include/cubit_b200.h.
extern "C" int cubit_decode_batch_static(cubit_ctx* ctx, int device_slot, const void* words, uint64_t n, uint16_t* form,
                                         uint32_t* slots, uint32_t* ctrl, cubit_counts* counts) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (counts) memset(counts, 0, sizeof *counts);
    if (ctx->devs.empty()) return fail(ctx, CUBIT_ERR_NO_DEVICE, "decode needs a CUDA device; this context has none");
    if (device_slot < 0 || (size_t)device_slot >= ctx->devs.size()) return fail(ctx, CUBIT_ERR_INVALID, "device_slot out of range");
    if (n > kStaticMaxWords)
        return fail(ctx, CUBIT_ERR_INVALID, "batch exceeds CUBIT_STATIC_MAX_WORDS (65536 words), the capacity of the built-in "
                                            "scratch; split it or use cubit_decode_batch");
    if (n == 0) return CUBIT_OK;
    if (!words || !form || !slots || !ctrl) return fail(ctx, CUBIT_ERR_INVALID, "null buffer");
    DeviceState* d = ctx->devs[(size_t)device_slot].get();
    if (d->device < 0 || d->device >= kMaxStaticDevices)
        return fail(ctx, CUBIT_ERR_INVALID, "device ordinal beyond what the built-in scratch is tracked for");
    // The array exists once per GPU for the whole process, whatever the number of contexts: its
    // lock is per device ordinal.  The context's staging lock guards the stream used below.
    std::lock_guard<std::mutex> scratch_lock(g_static_mu[d->device]);
    std::lock_guard<std::mutex> lock(d->stage_mu);
    CU_TRY(ctx, cudaSetDevice(d->device));
    if (!g_static_addr[d->device]) {
        // One-time set-up per device, with that device current: the symbol's address there.
        unsigned char* p = nullptr;
        CU_TRY(ctx, cudaGetSymbolAddress((void**)&p, g_static_scratch));
        g_static_addr[d->device] = p;
    }
    unsigned char* st = g_static_addr[d->device];
    unsigned long long* dc = (unsigned long long*)(st + kStaticCountersOff);
    unsigned long long host_counts[CNT_WORDS] = {0, 0, 0, 0, 0};
    // The array keeps what the previous call left: the counters are accumulated into, so they
    // are cleared; the record planes are fully overwritten for the first n entries.
    cudaError_t e = cudaMemsetAsync(dc, 0, sizeof host_counts, d->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(st, words, n * 16, cudaMemcpyHostToDevice, d->stream);
    if (e == cudaSuccess) {
        launch_decode(d, d->stream, (const uint4*)st, n, (uint16_t*)(st + kStaticFormOff), (uint32_t*)(st + kStaticSlotsOff), n,
                      (uint32_t*)(st + kStaticCtrlOff), dc);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(form, st + kStaticFormOff, n * 2, cudaMemcpyDeviceToHost, d->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(slots, st + kStaticSlotsOff, n * 32, cudaMemcpyDeviceToHost, d->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(ctrl, st + kStaticCtrlOff, n * 4, cudaMemcpyDeviceToHost, d->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_counts, dc, sizeof host_counts, cudaMemcpyDeviceToHost, d->stream);
    // Also after an error: copies already queued may still be writing into the caller's buffers or host_counts.
    const cudaError_t waited = cudaStreamSynchronize(d->stream);
    if (e == cudaSuccess) e = waited;
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, CUBIT_ERR_CUDA, std::string("static decode: ") + cudaGetErrorString(e));
    }
    if (counts) add_counts(counts, host_counts);
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

// ---- exported: cubin ----------------------------------------------------------------------------

extern "C" int cubit_elf_parse(const void* bytes, uint64_t len, cubit_elf** out) try {
    if (!bytes || !out) return fail(nullptr, CUBIT_ERR_INVALID, "bad argument");
    *out = nullptr;
    std::unique_ptr<cubit_elf> e(new cubit_elf);
    e->bytes = (const uint8_t*)bytes;
    e->len = len;
    try {
        e->text = elf_text_sections(e->bytes, len);
    } catch (const std::exception& ex) {
        return fail(nullptr, CUBIT_ERR_ELF, ex.what());
    }
    *out = e.release();
    return CUBIT_OK;
} catch (...) {
    return translate_exception(nullptr);
}

extern "C" void cubit_elf_free(cubit_elf* elf) { delete elf; }

extern "C" uint32_t cubit_elf_num_text(const cubit_elf* elf) { return elf ? (uint32_t)elf->text.size() : 0; }

extern "C" int cubit_elf_text(const cubit_elf* elf, uint32_t index, const char** name, uint64_t* offset, uint64_t* size) try {
    if (!elf || index >= elf->text.size()) return fail(nullptr, CUBIT_ERR_INVALID, "text section index out of range");
    if (name) *name = elf->text[index].name.c_str();
    if (offset) *offset = elf->text[index].offset;
    if (size) *size = elf->text[index].size;
    return CUBIT_OK;
} catch (...) {
    return translate_exception(nullptr);
}

extern "C" int cubit_elf_find(const cubit_elf* elf, const char* kernel_name, uint32_t* index) try {
    if (!elf || !kernel_name || !index) return fail(nullptr, CUBIT_ERR_INVALID, "bad argument");
    for (size_t i = 0; i < elf->text.size(); ++i)
        if (elf->text[i].name.find(kernel_name) != std::string::npos) {
            *index = (uint32_t)i;
            return CUBIT_OK;
        }
    std::string names;
    for (const TextSection& t : elf->text) names += (names.empty() ? "\"" : ", \"") + t.name + "\"";
    return fail(nullptr, CUBIT_ERR_NOT_FOUND, std::string("kernel '") + kernel_name + "' not found. Available: [" + names + "]");
} catch (...) {
    return translate_exception(nullptr);
}

extern "C" int cubit_decode_elf(cubit_ctx* ctx, const cubit_elf* elf, const uint32_t* indices, uint32_t n_sections,
                                uint64_t* word_start, uint64_t capacity, uint16_t* form, uint32_t* slots,
                                uint32_t* ctrl, void* raw_words, cubit_counts* counts) try {
    if (!ctx || !elf || !word_start) return fail(ctx, CUBIT_ERR_INVALID, "bad argument");
    if (counts) memset(counts, 0, sizeof *counts);
    if (!indices) n_sections = (uint32_t)elf->text.size();
    // Per-kernel offset table: record index of each section's first word.
    struct Range { uint64_t file_off, words, rec; };
    std::vector<Range> ranges;
    uint64_t total = 0;
    for (uint32_t k = 0; k < n_sections; ++k) {
        const uint32_t si = indices ? indices[k] : k;
        if (si >= elf->text.size()) return fail(ctx, CUBIT_ERR_INVALID, "text section index out of range");
        const TextSection& t = elf->text[si];
        if (t.offset > elf->len || t.size > elf->len - t.offset)
            return fail(ctx, CUBIT_ERR_ELF, "text section " + t.name + " extends past end of file");
        word_start[k] = total;
        const uint64_t w = t.size / 16;
        // Sections that follow each other in the file are fetched with one copy.
        if (!ranges.empty() && ranges.back().file_off + ranges.back().words * 16 == t.offset && w)
            ranges.back().words += w;
        else if (w)
            ranges.push_back(Range{t.offset, w, total});
        total += w;
    }
    word_start[n_sections] = total;
    if (!form) return CUBIT_OK;
    if (ctx->devs.empty()) return fail(ctx, CUBIT_ERR_NO_DEVICE, "decode needs a CUDA device; this context has none");
    if (!slots || !ctrl) return fail(ctx, CUBIT_ERR_INVALID, "null buffer");
    if (capacity < total) return fail(ctx, CUBIT_ERR_INVALID, "output capacity below the number of words");
    if (total == 0) return CUBIT_OK;

    // Shard records over devices by cumulative word count.  The number of launches depends on the
    // number of words only (one per 4 Mi words of a device's share), never on the number of kernels.
    const size_t g = ctx->devs.size();
    return for_each_device(ctx, counts, [&](size_t k, cubit_counts* part) {
        uint64_t b, e;
        shard_range(total, g, k, &b, &e);
        if (b == e) return (int)CUBIT_OK;
        DeviceState* d = ctx->devs[k].get();
        std::lock_guard<std::mutex> lock(d->stage_mu);
        CU_TRY(ctx, cudaSetDevice(d->device));
        // The device's share of the records goes through the staging area chunk by chunk: each chunk gathers
        // its part of the text ranges, is decoded by one launch and copied out while the next one comes in.
        const RecordStage L(e - b);
        return pipeline_host_range(ctx, d, b, e, L.chunk, L.half, part, "cubin decode", [&](const ChunkIO& io) {
            cudaError_t err = cudaSuccess;
            for (const Range& r : ranges) {
                const uint64_t lo = std::max(io.at, r.rec), hi = std::min(io.at + io.items, r.rec + r.words);
                if (lo >= hi) continue;
                const uint8_t* src = elf->bytes + r.file_off + (lo - r.rec) * 16;
                err = cudaMemcpyAsync(io.stage + (lo - io.at) * 16, src, (hi - lo) * 16, cudaMemcpyHostToDevice, io.stream);
                if (err != cudaSuccess) return err;
            }
            launch_decode(d, io.stream, (const uint4*)io.stage, io.items, (uint16_t*)(io.stage + L.o_form),
                          (uint32_t*)(io.stage + L.o_slots), L.chunk, (uint32_t*)(io.stage + L.o_ctrl), io.counters);
            err = cudaGetLastError();
            if (err == cudaSuccess) err = records_to_host(L, io, io.at, capacity, form, slots, ctrl);
            if (err == cudaSuccess && raw_words)
                err = cudaMemcpyAsync((uint8_t*)raw_words + io.at * 16, io.stage, io.items * 16, cudaMemcpyDeviceToHost, io.stream);
            return err;
        });
    });
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_infer_kernel_meta(cubit_ctx* ctx, const cubit_elf* elf, const uint32_t* indices, uint32_t n_sections,
                                       cubit_kernel_meta* meta, uint32_t* exit_offsets, uint64_t exit_capacity,
                                       uint64_t* n_exits) try {
    if (!ctx || !elf || !meta || !n_exits) return fail(ctx, CUBIT_ERR_INVALID, "bad argument");
    *n_exits = 0;
    if (ctx->devs.empty()) return fail(ctx, CUBIT_ERR_NO_DEVICE, "metadata inference needs a CUDA device; this context has none");
    if (!indices) n_sections = (uint32_t)elf->text.size();
    if (n_sections == 0) return CUBIT_OK;
    struct Range { uint64_t file_off, words, rec; };
    std::vector<Range> ranges;
    std::vector<uint64_t> start(n_sections + 1, 0);
    uint64_t total = 0;
    for (uint32_t k = 0; k < n_sections; ++k) {
        const uint32_t si = indices ? indices[k] : k;
        if (si >= elf->text.size()) return fail(ctx, CUBIT_ERR_INVALID, "text section index out of range");
        const TextSection& t = elf->text[si];
        if (t.offset > elf->len || t.size > elf->len - t.offset)
            return fail(ctx, CUBIT_ERR_ELF, "text section " + t.name + " extends past end of file");
        start[k] = total;
        const uint64_t w = t.size / 16;
        if (!ranges.empty() && ranges.back().file_off + ranges.back().words * 16 == t.offset && w) ranges.back().words += w;
        else if (w) ranges.push_back(Range{t.offset, w, total});
        total += w;
    }
    start[n_sections] = total;
    std::vector<uint32_t> max_reg(n_sections, 0), barriers(n_sections, 0);
    std::vector<uint8_t> flags(total, 0);
    if (total) {
        // One device: the per-kernel reduction is tiny next to a decode.
        DeviceState* d = ctx->devs[0].get();
        std::lock_guard<std::mutex> lock(d->stage_mu);
        CU_TRY(ctx, cudaSetDevice(d->device));
        const uint64_t o_start = align_up(total * 16, 256), o_max = o_start + align_up((n_sections + 1) * 8, 256);
        const uint64_t o_bar = o_max + align_up(n_sections * 4, 256), o_flag = o_bar + align_up(n_sections * 4, 256);
        int rc = ensure_stage(ctx, d, o_flag + total);
        if (rc) return rc;
        uint8_t* st = (uint8_t*)d->stage;
        for (const Range& r : ranges)
            CU_TRY_DRAIN(ctx, d->stream, cudaMemcpyAsync(st + r.rec * 16, elf->bytes + r.file_off, r.words * 16, cudaMemcpyHostToDevice, d->stream));
        CU_TRY_DRAIN(ctx, d->stream, cudaMemcpyAsync(st + o_start, start.data(), (n_sections + 1) * 8, cudaMemcpyHostToDevice, d->stream));
        CU_TRY_DRAIN(ctx, d->stream, cudaMemsetAsync(st + o_max, 0, o_flag - o_max, d->stream));
        if (use_shared(d, total))
            meta_kernel<HotShared><<<grid_shared(d, total), kBlockShared, d->hot_bytes, d->stream>>>(
                d->view, (const uint4*)st, total, (const uint64_t*)(st + o_start), n_sections, (uint32_t*)(st + o_max),
                (uint32_t*)(st + o_bar), st + o_flag);
        else
            meta_kernel<HotGlobal><<<grid_for(d, total), kBlock, 0, d->stream>>>(
                d->view, (const uint4*)st, total, (const uint64_t*)(st + o_start), n_sections, (uint32_t*)(st + o_max),
                (uint32_t*)(st + o_bar), st + o_flag);
        CU_TRY_DRAIN(ctx, d->stream, cudaGetLastError());
        CU_TRY_DRAIN(ctx, d->stream, cudaMemcpyAsync(max_reg.data(), st + o_max, n_sections * 4, cudaMemcpyDeviceToHost, d->stream));
        CU_TRY_DRAIN(ctx, d->stream, cudaMemcpyAsync(barriers.data(), st + o_bar, n_sections * 4, cudaMemcpyDeviceToHost, d->stream));
        CU_TRY_DRAIN(ctx, d->stream, cudaMemcpyAsync(flags.data(), st + o_flag, total, cudaMemcpyDeviceToHost, d->stream));
        CU_TRY_DRAIN(ctx, d->stream, cudaStreamSynchronize(d->stream));
    }
    uint64_t ne = 0;
    for (uint32_t k = 0; k < n_sections; ++k) {
        cubit_kernel_meta& m = meta[k];
        m.max_reg = max_reg[k];
        m.barrier_mask = barriers[k];
        m.regcount = std::max<uint32_t>((max_reg[k] + 32) & ~31u, 32);   // registers come in blocks of 32
        m.num_barriers = (uint32_t)__builtin_popcount(barriers[k]);
        m.first_exit = ne;
        m.n_exits = 0;
        for (uint64_t i = start[k]; i < start[k + 1]; ++i)
            if (flags[i]) {
                if (exit_offsets && ne < exit_capacity) exit_offsets[ne] = (uint32_t)((i - start[k]) * 16);
                ++ne; ++m.n_exits;
            }
    }
    *n_exits = ne;
    if (exit_offsets && ne > exit_capacity) return fail(ctx, CUBIT_ERR_INVALID, "exit_offsets capacity below the number of EXIT instructions");
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_elf_build(const char* const* names, const void* const* code, const uint64_t* code_bytes,
                               uint32_t n_kernels, void* out, uint64_t capacity, uint64_t* out_len) try {
    if (!out_len || (n_kernels && (!names || !code || !code_bytes))) return fail(nullptr, CUBIT_ERR_INVALID, "bad argument");
    std::vector<BuildKernel> ks;
    for (uint32_t k = 0; k < n_kernels; ++k) ks.push_back(BuildKernel{names[k], (const uint8_t*)code[k], code_bytes[k]});
    try {
        *out_len = elf_build(ks, (uint8_t*)out, capacity);
    } catch (const std::exception& e) {
        return fail(nullptr, CUBIT_ERR_ELF, e.what());
    }
    return CUBIT_OK;
} catch (...) {
    return translate_exception(nullptr);
}

// ---- SASS text ---------------------------------------------------------------------------

namespace {

void put_bits(uint32_t slots[8], uint32_t pos, uint32_t nbits, uint64_t v) {
    for (uint32_t done = 0; done < nbits;) {
        const uint32_t limb = (pos + done) >> 5, off = (pos + done) & 31u;
        const uint32_t take = std::min(32u - off, nbits - done);
        const uint32_t mask = take == 32u ? 0xFFFFFFFFu : ((1u << take) - 1u);
        slots[limb] = (slots[limb] & ~(mask << off)) | (((uint32_t)(v >> done) & mask) << off);
        done += take;
    }
}

struct LoweredBatch {
    std::vector<uint16_t> form;
    std::vector<uint32_t> slots;   // 8 per instruction, instruction-major here
    std::vector<uint32_t> ctrl;
    std::vector<u128> clear, set;
};

// Host threads for the text layer: printing and lowering are per-instruction and independent.
unsigned text_threads(uint64_t n) {
    const unsigned hw = std::max(1u, std::thread::hardware_concurrency());
    return (unsigned)std::min<uint64_t>(std::min(hw, 64u), std::max<uint64_t>(1, n / 2048));
}

// Runs fn(begin, end, part) over `parts` contiguous ranges of [0, n), one host thread each.
// An exception in a range is rethrown here; with several, the one of the lowest range.
template <typename Fn>
void parallel_ranges(uint64_t n, unsigned parts, Fn fn) {
    if (parts <= 1) { fn((uint64_t)0, n, 0u); return; }
    std::vector<std::exception_ptr> errors(parts);
    std::vector<std::thread> pool;
    for (unsigned k = 0; k < parts; ++k)
        pool.emplace_back([&, k] {
            try {
                fn(n * k / parts, n * (k + 1) / parts, k);
            } catch (...) {
                errors[k] = std::current_exception();
            }
        });
    for (std::thread& th : pool) th.join();
    for (const std::exception_ptr& e : errors)
        if (e) std::rethrow_exception(e);
}

// One instruction -> record + patch appended to `out`.  Throws TextError carrying the message the
// reference would report.
void lower_one(const cubit_ctx* ctx, const TextInstruction& insn, int mode, LoweredBatch* out) {
    LoweredInstruction low;
    try {
        low = ctx->text->lower(insn);
    } catch (const TextError& e) {
        if (mode == CUBIT_TEXT_ONE) throw TextError(std::string("encode error: ") + e.what());
        char at[32];
        snprintf(at, sizeof at, "0x%x", insn.addr);
        throw TextError(std::string("encode error at addr ") + at + ": " + e.what());
    }
    uint32_t slots[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (!low.raw) {
        const VariantMeta& m = ctx->flat.meta[low.variant];
        for (size_t k = 0; k < m.fields.size(); ++k) {
            const FieldMeta& f = m.fields[k];
            if (f.dst_pos == 0xFFFFFFFFu) continue;
            put_bits(slots, f.dst_pos, f.stored_bits, low.values[k]);
        }
    }
    out->form.push_back(low.raw ? (uint16_t)0xFFFF : (uint16_t)low.variant);
    out->slots.insert(out->slots.end(), slots, slots + 8);
    out->ctrl.push_back(low.ctrl);
    out->clear.push_back(low.clear);
    out->set.push_back(low.set);
}

void append_batch(LoweredBatch* to, const LoweredBatch& from) {
    to->form.insert(to->form.end(), from.form.begin(), from.form.end());
    to->slots.insert(to->slots.end(), from.slots.begin(), from.slots.end());
    to->ctrl.insert(to->ctrl.end(), from.ctrl.begin(), from.ctrl.end());
    to->clear.insert(to->clear.end(), from.clear.begin(), from.clear.end());
    to->set.insert(to->set.end(), from.set.begin(), from.set.end());
}

void lower_text(const cubit_ctx* ctx, const char* text, uint32_t base_addr, int mode, LoweredBatch* out) {
    if (mode == CUBIT_TEXT_ONE) {
        TextInstruction insn;
        try {
            insn = parse_sass(text, base_addr);
        } catch (const TextError& e) {
            throw TextError(std::string("parse error: ") + e.what());
        }
        lower_one(ctx, insn, mode, out);
        return;
    }
    // Statements are split and labels resolved in one sequential pass; lowering runs in parallel
    // and reports the failure of the earliest statement, as a sequential pass would.
    const RangeRunner runner = [](size_t n, const std::function<void(size_t, size_t)>& body) {
        parallel_ranges(n, text_threads(n), [&](uint64_t b, uint64_t e, unsigned) { body((size_t)b, (size_t)e); });
    };
    const std::vector<TextInstruction> insns = parse_program(text, base_addr, runner);
    const unsigned parts = text_threads(insns.size());
    std::vector<LoweredBatch> piece(parts);
    parallel_ranges(insns.size(), parts, [&](uint64_t b, uint64_t e, unsigned k) {
        for (uint64_t i = b; i < e; ++i) lower_one(ctx, insns[i], mode, &piece[k]);
    });
    for (const LoweredBatch& p : piece) append_batch(out, p);
}

void json_escape(const std::string& s, std::string* out) {
    *out += '"';
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { *out += '\\'; *out += (char)c; }
        else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); *out += b; }
        else *out += (char)c;
    }
    *out += '"';
}

}  // namespace

extern "C" int cubit_text_lower(cubit_ctx* ctx, const char* text, uint32_t base_addr, int mode, uint64_t capacity,
                                uint16_t* form, uint32_t* slots, uint32_t* ctrl, void* clear, void* set,
                                uint64_t* n_out) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (!text || !n_out) return fail(ctx, CUBIT_ERR_INVALID, "null argument");
    if (mode != CUBIT_TEXT_ONE && mode != CUBIT_TEXT_PROGRAM) return fail(ctx, CUBIT_ERR_INVALID, "unknown text mode");
    LoweredBatch b;
    try {
        lower_text(ctx, text, base_addr, mode, &b);
    } catch (const TextError& e) {
        return fail(ctx, CUBIT_ERR_TEXT, e.what());
    } catch (const std::exception& e) {
        return fail(ctx, CUBIT_ERR_INVALID, e.what());
    }
    const uint64_t n = b.form.size();
    *n_out = n;
    if (n > capacity || !form || !slots || !ctrl || !clear || !set) return CUBIT_OK;
    for (uint64_t i = 0; i < n; ++i) {
        form[i] = b.form[i];
        ctrl[i] = b.ctrl[i];
        for (int s = 0; s < 8; ++s) slots[(uint64_t)s * capacity + i] = b.slots[i * 8 + s];
        memcpy((uint8_t*)clear + i * 16, &b.clear[i], 16);
        memcpy((uint8_t*)set + i * 16, &b.set[i], 16);
    }
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_text_encode(cubit_ctx* ctx, const char* text, uint32_t base_addr, int mode, uint64_t capacity,
                                 void* words, uint64_t* n_out) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (!text || !n_out) return fail(ctx, CUBIT_ERR_INVALID, "null argument");
    if (mode != CUBIT_TEXT_ONE && mode != CUBIT_TEXT_PROGRAM) return fail(ctx, CUBIT_ERR_INVALID, "unknown text mode");
    LoweredBatch b;
    try {
        lower_text(ctx, text, base_addr, mode, &b);
    } catch (const TextError& e) {
        return fail(ctx, CUBIT_ERR_TEXT, e.what());
    } catch (const std::exception& e) {
        return fail(ctx, CUBIT_ERR_INVALID, e.what());
    }
    const uint64_t n = b.form.size();
    *n_out = n;
    if (n > capacity || !words || n == 0) return CUBIT_OK;
    std::vector<uint32_t> planes(8 * n);
    for (uint64_t i = 0; i < n; ++i)
        for (int s = 0; s < 8; ++s) planes[(uint64_t)s * n + i] = b.slots[i * 8 + s];
    const int rc = cubit_encode_batch(ctx, b.form.data(), planes.data(), b.ctrl.data(), n, words, CUBIT_MEM_HOST, nullptr);
    if (rc) return rc;
    for (uint64_t i = 0; i < n; ++i) {
        u128 w;
        memcpy(&w, (uint8_t*)words + i * 16, 16);
        w = (w & ~b.clear[i]) | b.set[i];
        memcpy((uint8_t*)words + i * 16, &w, 16);
    }
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_text_parse(cubit_ctx* ctx, const char* line, uint32_t addr, char* json, uint64_t capacity,
                                uint64_t* needed) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (!line || !needed) return fail(ctx, CUBIT_ERR_INVALID, "null argument");
    TextInstruction insn;
    try {
        insn = parse_cuasm_line(line, addr);
    } catch (const TextError& e) {
        return fail(ctx, CUBIT_ERR_TEXT, std::string("parse error: ") + e.what());
    }
    static const char* const kKinds[] = {"Reg", "UReg", "Pred", "UPred", "Imm32", "Imm64", "FloatImm", "Addr",
                                         "ConstMem", "Desc", "BranchTarget", "Barrier", "SysReg", "Label"};
    std::string j = "{\"key\":";
    json_escape(insn.key, &j);
    j += ",\"opcode\":"; json_escape(insn.opcode, &j);
    j += ",\"opcode_full\":"; json_escape(insn.opcode_full, &j);
    j += ",\"mod_group\":"; json_escape(extract_mod_group(insn.raw_text), &j);
    j += ",\"addr\":" + std::to_string(insn.addr);
    if (insn.has_guard)
        j += std::string(",\"guard\":{\"pred\":") + std::to_string((int)insn.guard_pred) + ",\"negated\":" +
             (insn.guard_neg ? "true" : "false") + ",\"uniform\":" + (insn.guard_uniform ? "true" : "false") + "}";
    else j += ",\"guard\":null";
    j += ",\"modifiers\":[";
    for (size_t k = 0; k < insn.modifiers.size(); ++k) { if (k) j += ','; json_escape(insn.modifiers[k], &j); }
    j += "],\"ctrl\":"; json_escape(format_control_code(insn.ctrl), &j);
    j += std::string(",\"hand_sched\":") + (insn.hand_sched ? "true" : "false");
    j += ",\"operands\":[";
    auto b = [](bool v) { return v ? "true" : "false"; };
    for (size_t k = 0; k < insn.operands.size(); ++k) {
        const TextOperand& op = insn.operands[k];
        if (k) j += ',';
        j += std::string("{\"type\":\"") + operand_type_label(op) + "\",\"kind\":\"" + kKinds[(size_t)op.kind] + "\"";
        switch (op.kind) {
            case OperandKind::Reg:
                j += ",\"num\":" + std::to_string((int)op.num) + ",\"neg\":" + b(op.neg) + ",\"abs\":" + b(op.abs) +
                     ",\"inv\":" + b(op.inv) + ",\"reuse\":" + b(op.reuse);
                break;
            case OperandKind::UReg:
                j += ",\"num\":" + std::to_string((int)op.num) + ",\"neg\":" + b(op.neg) + ",\"reuse\":" + b(op.reuse) +
                     ",\"is_zero\":" + b(op.is_zero);
                break;
            case OperandKind::Pred: case OperandKind::UPred:
                j += ",\"num\":" + std::to_string((int)op.num) + ",\"neg\":" + b(op.neg);
                break;
            case OperandKind::Imm32: j += ",\"value\":" + std::to_string((long long)op.imm); break;
            case OperandKind::Imm64: case OperandKind::FloatImm:
                j += ",\"bits\":" + std::to_string((unsigned long long)op.bits);
                break;
            case OperandKind::Addr: case OperandKind::ConstMem: case OperandKind::Desc:
                j += std::string(",\"base_reg\":") + (op.has_base ? std::to_string((int)op.base) : "null");
                if (op.kind != OperandKind::Desc) j += std::string(",\"ur_reg\":") + (op.has_ur ? std::to_string((int)op.ur) : "null");
                if (op.kind == OperandKind::Desc) j += ",\"ur_idx\":" + std::to_string((int)op.ur_idx);
                if (op.kind == OperandKind::ConstMem) j += ",\"bank\":" + std::to_string((int)op.bank);
                if (op.kind != OperandKind::ConstMem) {
                    j += ",\"base_reg_suffix\":";
                    if (op.has_suffix) json_escape(op.suffix, &j); else j += "null";
                }
                j += ",\"offset\":" + std::to_string((long long)op.offset);
                break;
            case OperandKind::BranchTarget: j += ",\"target\":" + std::to_string(op.target); break;
            case OperandKind::Barrier: j += ",\"num\":" + std::to_string((int)op.num); break;
            case OperandKind::SysReg: case OperandKind::Label: j += ",\"text\":"; json_escape(op.text, &j); break;
        }
        j += '}';
    }
    j += "]}";
    *needed = j.size() + 1;
    if (json && capacity >= j.size() + 1) memcpy(json, j.c_str(), j.size() + 1);
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

namespace {

uint64_t get_bits(const uint32_t slots[8], uint32_t pos, uint32_t nbits) {
    uint64_t v = 0;
    for (uint32_t done = 0; done < nbits;) {
        const uint32_t limb = (pos + done) >> 5, off = (pos + done) & 31u;
        const uint32_t take = std::min(32u - off, nbits - done);
        const uint64_t mask = take == 32u ? 0xFFFFFFFFull : ((1ull << take) - 1ull);
        v |= (((uint64_t)slots[limb] >> off) & mask) << done;
        done += take;
    }
    return v;
}

// The printer's view of one decoded record (reference src/decoder.rs:289-381).
DecodedView view_of_record(const cubit_ctx* ctx, uint32_t form, const uint32_t slots[8], uint32_t ctrl, u128 raw,
                           uint32_t addr) {
    const VariantMeta& m = ctx->flat.meta[form];
    DecodedView v;
    v.key = m.key; v.mod_group = m.mod_group; v.opcode = m.opcode; v.raw = raw; v.addr = addr;
    v.cache = &ctx->print_cache[form];
    v.fields.reserve(m.fields.size() + 4);
    for (const FieldMeta& f : m.fields) {
        PrintField pf;
        pf.shift = f.shift; pf.bits = f.bits; pf.token_idx = f.token_idx; pf.ext = f.extraction;
        pf.value = f.dst_pos == 0xFFFFFFFFu ? 0 : get_bits(slots, f.dst_pos, f.stored_bits);
        v.fields.push_back(std::move(pf));
    }
    static const struct { uint32_t bit; bool rb; const char* ext; } kSynth[4] = {
        {63, true, "neg"}, {62, true, "abs"}, {72, false, "neg"}, {73, false, "abs"}};
    for (int k = 0; k < 4; ++k)
        if ((ctrl >> (24 + k)) & 1u) {
            PrintField pf;
            pf.shift = kSynth[k].bit; pf.bits = 1; pf.value = 1; pf.ext = kSynth[k].ext;
            pf.token_idx = kSynth[k].rb ? m.rb_tok : m.ra_tok;
            v.fields.push_back(std::move(pf));
        }
    return v;
}

std::string hex_word(u128 w) {
    char buf[40];
    snprintf(buf, sizeof buf, "%016llx%016llx", (unsigned long long)(uint64_t)(w >> 64), (unsigned long long)(uint64_t)w);
    return buf;
}

// Decodes when the caller has no records; returns the records either way.
int records_for_print(cubit_ctx* ctx, const void* words, uint64_t n, const uint16_t*& form, const uint32_t*& slots,
                      const uint32_t*& ctrl, std::vector<uint16_t>* f, std::vector<uint32_t>* s, std::vector<uint32_t>* c) {
    if (form && slots && ctrl) return CUBIT_OK;
    if (form || slots || ctrl) return fail(ctx, CUBIT_ERR_INVALID, "pass form, slots and ctrl together, or none of them");
    f->resize(n); s->resize(8 * n); c->resize(n);
    const int rc = cubit_decode_batch(ctx, words, n, f->data(), s->data(), c->data(), nullptr, CUBIT_MEM_HOST, nullptr);
    form = f->data(); slots = s->data(); ctrl = c->data();
    return rc;
}

std::string print_word(const cubit_ctx* ctx, const uint8_t* words, uint64_t i, uint64_t n, uint32_t addr,
                       const uint16_t* form, const uint32_t* slots, const uint32_t* ctrl) {
    u128 raw;
    memcpy(&raw, words + i * 16, 16);
    if (form[i] == 0xFFFFu || form[i] >= ctx->flat.meta.size()) return "/* ? 0x" + hex_word(raw) + " */";
    uint32_t sl[8];
    for (int k = 0; k < 8; ++k) sl[k] = slots[(uint64_t)k * n + i];
    return to_sass(view_of_record(ctx, form[i], sl, ctrl[i], raw, addr));
}

}  // namespace

extern "C" int cubit_text_print(cubit_ctx* ctx, const void* words, uint64_t n, uint32_t base_addr, const uint16_t* form,
                                const uint32_t* slots, const uint32_t* ctrl, char* out, uint64_t capacity,
                                uint64_t* needed) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (!needed || (n && !words)) return fail(ctx, CUBIT_ERR_INVALID, "null argument");
    std::vector<uint16_t> f;
    std::vector<uint32_t> s, c;
    if (n) {
        const int rc = records_for_print(ctx, words, n, form, slots, ctrl, &f, &s, &c);
        if (rc) return rc;
    }
    const unsigned parts = text_threads(n);
    std::vector<std::string> piece(parts);
    parallel_ranges(n, parts, [&](uint64_t b, uint64_t e, unsigned k) {
        for (uint64_t i = b; i < e; ++i) {
            piece[k] += print_word(ctx, (const uint8_t*)words, i, n, base_addr + (uint32_t)(16 * i), form, slots, ctrl);
            piece[k] += '\n';
        }
    });
    std::string text;
    for (const std::string& p : piece) text += p;
    *needed = text.size() + 1;
    if (out && capacity >= text.size() + 1) memcpy(out, text.c_str(), text.size() + 1);
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

// ---- listings ------------------------------------------------------------------------------

namespace {

// Lowers the printed text of every decodable word (in parallel); `where` lists, in order, the
// words whose text parsed and found a table entry, `out` their records and patches.
void lower_printed(const cubit_ctx* ctx, const std::vector<std::string>& text, const std::vector<uint8_t>& unknown,
                   const std::vector<uint32_t>& addr_of, LoweredBatch* out, std::vector<uint64_t>* where) {
    const uint64_t total = text.size();
    const unsigned parts = text_threads(total);
    std::vector<LoweredBatch> piece(parts);
    std::vector<std::vector<uint64_t>> piece_where(parts);
    parallel_ranges(total, parts, [&](uint64_t b, uint64_t e, unsigned k) {
        for (uint64_t i = b; i < e; ++i) {
            if (unknown[i]) continue;
            try {
                lower_one(ctx, parse_sass(text[i], addr_of[i]), CUBIT_TEXT_ONE, &piece[k]);
                piece_where[k].push_back(i);
            } catch (const TextError&) {
                // does not parse, or no table entry fits
            }
        }
    });
    for (unsigned k = 0; k < parts; ++k) {
        append_batch(out, piece[k]);
        where->insert(where->end(), piece_where[k].begin(), piece_where[k].end());
    }
}

std::string strip_statement_end(std::string t) {
    while (t.size() >= 2 && t.compare(t.size() - 2, 2, " ;") == 0) t.erase(t.size() - 2);
    while (!t.empty() && t.back() == ';') t.pop_back();
    return t;
}

// Mnemonic without guard and modifiers (reference src/main.rs:506-513).
std::string listing_opcode(const std::string& text) {
    size_t b = 0, e = text.size();
    while (b < e && isspace((unsigned char)text[b])) ++b;
    while (e > b && isspace((unsigned char)text[e - 1])) --e;
    std::string t = text.substr(b, e - b);
    if (!t.empty() && t[0] == '@') {
        size_t ws = 1;
        while (ws < t.size() && !isspace((unsigned char)t[ws])) ++ws;
        t = ws < t.size() ? t.substr(ws + 1) : std::string();
    }
    b = 0;
    while (b < t.size() && isspace((unsigned char)t[b])) ++b;
    size_t k = b;
    while (k < t.size() && !isspace((unsigned char)t[k]) && t[k] != '.') ++k;
    return t.substr(b, k - b);
}
bool listing_is_branch(const std::string& text) {
    const std::string op = listing_opcode(text);
    return op == "BRA" || op == "JMP" || op == "CALL" || op == "BRX" || op == "BSSY" || op == "BSYNC";
}
// Value of the last "0x<hex>" in the text that fits 32 bits: a branch's target operand.
bool listing_last_hex(const std::string& t, uint32_t* out) {
    bool found = false;
    for (size_t i = 0; i + 2 < t.size(); ++i) {
        if (t[i] != '0' || t[i + 1] != 'x') continue;
        size_t k = i + 2;
        uint64_t v = 0;
        bool fits = true;
        while (k < t.size() && isxdigit((unsigned char)t[k])) {
            const char c = t[k];
            v = v * 16 + (uint64_t)(isdigit((unsigned char)c) ? c - '0' : (tolower(c) - 'a' + 10));
            if (v > 0xFFFFFFFFull) fits = false;
            ++k;
        }
        if (k == i + 2) continue;
        if (fits) { *out = (uint32_t)v; found = true; }
        i = k - 1;
    }
    return found;
}
// Largest n of any whole-word "R<n>" other than 255, at least `floor`.
uint32_t listing_max_reg(const std::string& t, uint32_t floor) {
    uint32_t best = floor;
    auto wordc = [](char c) { return isalnum((unsigned char)c) || c == '_'; };
    for (size_t i = 0; i < t.size(); ++i) {
        if (t[i] != 'R' || (i > 0 && wordc(t[i - 1]))) continue;
        size_t k = i + 1;
        uint64_t v = 0;
        while (k < t.size() && isdigit((unsigned char)t[k]) && v < (1ull << 40)) v = v * 10 + (uint64_t)(t[k++] - '0');
        while (k < t.size() && isdigit((unsigned char)t[k])) ++k;
        if (k == i + 1 || (k < t.size() && wordc(t[k]))) continue;
        if (v <= 0xFFFFFFFFull && v != 255 && v > best) best = (uint32_t)v;
    }
    return best;
}

struct KernelInfo { uint32_t shared_size = 0; std::vector<std::pair<uint32_t, uint32_t>> params; };

// Shared-memory size and parameter list from .nv.shared.<k> / .nv.info.<k> (reference src/main.rs:423-479).
KernelInfo kernel_info(const cubit_elf* elf, const std::vector<ElfSection>& sections, const std::string& kernel) {
    KernelInfo info;
    for (const ElfSection& s : sections)
        if (s.name == ".nv.shared." + kernel) {
            if (s.size > 0) info.shared_size = (uint32_t)s.size;
            break;
        }
    for (const ElfSection& s : sections) {
        if (s.name != ".nv.info." + kernel) continue;
        if (s.offset <= elf->len && s.size <= elf->len - s.offset) {
            const uint8_t* data = elf->bytes + s.offset;
            uint64_t pos = 0;
            while (pos + 4 <= s.size) {
                const uint8_t fmt = data[pos], attr = data[pos + 1];
                const uint64_t dsz = (uint64_t)data[pos + 2] | ((uint64_t)data[pos + 3] << 8);
                pos += 4;
                if (pos + dsz > s.size) break;
                const uint8_t* p = data + pos;
                auto u32at = [&](uint64_t o) { return (uint32_t)p[o] | ((uint32_t)p[o + 1] << 8) | ((uint32_t)p[o + 2] << 16) | ((uint32_t)p[o + 3] << 24); };
                if (fmt == 0x04 && attr == 0x08 && dsz >= 4 && info.shared_size == 0) {
                    const uint32_t v = u32at(0);
                    if (v > 0) info.shared_size = v;
                }
                if (fmt == 0x04 && attr == 0x17 && dsz >= 12)
                    info.params.push_back({(uint32_t)p[4] | ((uint32_t)p[5] << 8), u32at(8) >> 18});
                pos += dsz;
            }
        }
        break;
    }
    return info;
}

}  // namespace

extern "C" int cubit_disassemble(cubit_ctx* ctx, const cubit_elf* elf, const char* only_kernel, int frozen, char* out,
                                 uint64_t capacity, uint64_t* needed, uint64_t* n_raw) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (!elf || !needed) return fail(ctx, CUBIT_ERR_INVALID, "null argument");
    if (n_raw) *n_raw = 0;
    std::vector<ElfSection> sections;
    try {
        sections = elf_sections(elf->bytes, elf->len);
    } catch (const std::exception& e) {
        return fail(ctx, CUBIT_ERR_ELF, e.what());
    }
    // The chosen kernels, then one decode over all their words.
    std::vector<uint32_t> chosen;
    std::vector<std::string> names;
    for (uint32_t i = 0; i < elf->text.size(); ++i) {
        const std::string& sec = elf->text[i].name;
        const std::string kernel = sec.compare(0, 6, ".text.") == 0 ? sec.substr(6) : sec;
        if (only_kernel && kernel != only_kernel) continue;
        chosen.push_back(i);
        names.push_back(kernel);
    }
    std::vector<uint64_t> start(chosen.size() + 1, 0);
    std::vector<uint16_t> form;
    std::vector<uint32_t> slots, ctrl;
    std::vector<uint8_t> words;
    uint64_t total = 0;
    if (!chosen.empty()) {
        int rc = cubit_decode_elf(ctx, elf, chosen.data(), (uint32_t)chosen.size(), start.data(), 0, nullptr, nullptr,
                                  nullptr, nullptr, nullptr);
        if (rc) return rc;
        total = start.back();
        form.resize(total); slots.resize(8 * total); ctrl.resize(total); words.resize(16 * total);
        if (total) {
            rc = cubit_decode_elf(ctx, elf, chosen.data(), (uint32_t)chosen.size(), start.data(), total, form.data(),
                                  slots.data(), ctrl.data(), words.data(), nullptr);
            if (rc) return rc;
        }
    }
    std::vector<std::string> text(total);
    std::vector<uint8_t> unknown(total, 0);
    std::vector<uint32_t> addr_of(total);
    for (size_t k = 0; k < chosen.size(); ++k)
        for (uint64_t i = start[k]; i < start[k + 1]; ++i) addr_of[i] = (uint32_t)((i - start[k]) * 16);
    const unsigned parts = text_threads(total);
    parallel_ranges(total, parts, [&](uint64_t b, uint64_t e, unsigned) {
        for (uint64_t i = b; i < e; ++i) {
            unknown[i] = form[i] == 0xFFFFu;
            text[i] = strip_statement_end(print_word(ctx, words.data(), i, total, addr_of[i], form.data(), slots.data(), ctrl.data()));
        }
    });
    // Frozen listings keep only lines whose text encodes back to the same word outside the
    // scheduling field: lower every line on the host, encode all of them in one batch.
    std::vector<uint8_t> faithful(total, 0);
    if (frozen && total) {
        LoweredBatch b;
        std::vector<uint64_t> where;
        lower_printed(ctx, text, unknown, addr_of, &b, &where);
        const uint64_t m = where.size();
        if (m) {
            std::vector<uint32_t> planes(8 * m);
            for (uint64_t i = 0; i < m; ++i)
                for (int s = 0; s < 8; ++s) planes[(uint64_t)s * m + i] = b.slots[i * 8 + s];
            std::vector<uint8_t> enc(16 * m);
            const int rc = cubit_encode_batch(ctx, b.form.data(), planes.data(), b.ctrl.data(), m, enc.data(), CUBIT_MEM_HOST, nullptr);
            if (rc) return rc;
            const u128 keep = ~((u128)0x1FFFF << 105);
            for (uint64_t i = 0; i < m; ++i) {
                u128 e, w;
                memcpy(&e, enc.data() + i * 16, 16);
                memcpy(&w, words.data() + where[i] * 16, 16);
                e = (e & ~b.clear[i]) | b.set[i];
                faithful[where[i]] = ((e ^ w) & keep) == 0;
            }
        }
    }

    // Per-word line text, in parallel; per-kernel headers and the final join in order.
    std::vector<uint32_t> kernel_of(total);
    for (size_t k = 0; k < chosen.size(); ++k)
        for (uint64_t i = start[k]; i < start[k + 1]; ++i) kernel_of[i] = (uint32_t)k;
    // Frozen: branch targets and the largest register per word first (both read the text).
    std::vector<uint8_t> has_target(frozen ? total : 0, 0);
    std::vector<uint32_t> target(frozen ? total : 0, 0), word_max_reg(frozen ? total : 0, 1);
    if (frozen)
        parallel_ranges(total, parts, [&](uint64_t b, uint64_t e, unsigned) {
            for (uint64_t i = b; i < e; ++i) {
                uint32_t t;
                if (!unknown[i] && listing_is_branch(text[i]) && listing_last_hex(text[i], &t)) { has_target[i] = 1; target[i] = t; }
                word_max_reg[i] = listing_max_reg(text[i], 1);
            }
        });
    std::vector<std::vector<uint32_t>> targets(frozen ? chosen.size() : 0);
    std::vector<uint32_t> max_reg(chosen.size(), 1);
    if (frozen)
        for (size_t k = 0; k < chosen.size(); ++k) {
            for (uint64_t i = start[k]; i < start[k + 1]; ++i) {
                if (has_target[i]) targets[k].push_back(target[i]);
                max_reg[k] = std::max(max_reg[k], word_max_reg[i]);
            }
            std::sort(targets[k].begin(), targets[k].end());
        }
    std::vector<std::string> body(total);
    std::vector<uint64_t> raw_count(std::max(parts, 1u), 0);
    parallel_ranges(total, parts, [&](uint64_t b, uint64_t e, unsigned part) {
        char buf[96];
        for (uint64_t i = b; i < e; ++i) {
            const uint32_t addr = addr_of[i];
            u128 w;
            memcpy(&w, words.data() + i * 16, 16);
            if (!frozen) {
                snprintf(buf, sizeof buf, "  /*%04x*/  ", addr);
                if (unknown[i]) { body[i] = buf + text[i]; ++raw_count[part]; continue; }
                char tail[48];
                snprintf(tail, sizeof tail, " /* @sched 0x%05x */ ;", (uint32_t)((w >> 105) & 0x1FFFF));
                body[i] = buf + text[i] + tail;
                continue;
            }
            const std::vector<uint32_t>& tg = targets[kernel_of[i]];
            std::string label = "    ";
            if (std::binary_search(tg.begin(), tg.end(), addr)) {
                snprintf(buf, sizeof buf, "L_%x:  ", addr);
                label = buf;
            }
            if (unknown[i] || !faithful[i]) {
                body[i] = label + "__raw__0x" + hex_word(w) + " ;";
                ++raw_count[part];
                continue;
            }
            const std::string cc = format_control_code(unpack_control_code((uint32_t)((w >> 105) & 0x1FFFF)));
            std::string t = text[i];
            if (has_target[i]) {
                snprintf(buf, sizeof buf, "0x%x", target[i]);
                const size_t pos = t.rfind(buf);
                if (pos != std::string::npos) {
                    char lab[32];
                    snprintf(lab, sizeof lab, "L_%x", target[i]);
                    t.replace(pos, strlen(buf), lab);
                }
            }
            body[i] = label + "[" + cc + "] " + t + " ;";
        }
    });
    uint64_t raw_lines = 0;
    for (uint64_t c : raw_count) raw_lines += c;
    size_t bytes = 1;
    for (const std::string& l : body) bytes += l.size() + 1;
    std::string listing;
    listing.reserve(bytes + chosen.size() * 256);
    bool first_line = true;
    auto put = [&](const std::string& l) {
        if (!first_line) listing += '\n';
        listing += l;
        first_line = false;
    };
    for (size_t k = 0; k < chosen.size(); ++k) {
        if (!first_line) put("");
        const KernelInfo info = kernel_info(elf, sections, names[k]);
        if (frozen) {
            put(".entry " + names[k]);
            put("    .reg R0-R" + std::to_string(std::min(max_reg[k] + 4, 255u)));
            std::vector<std::pair<uint32_t, uint32_t>> params = info.params;
            std::stable_sort(params.begin(), params.end(), [](const auto& a, const auto& b) { return a.first < b.first; });
            for (size_t p = 0; p < params.size(); ++p)
                put(std::string("    .param ") + (params[p].second > 4 ? "u64" : "u32") + " p" + std::to_string(p));
        } else {
            put("// " + names[k]);
        }
        if (info.shared_size > 0) put("    .shared smem[" + std::to_string(info.shared_size) + "]");
        for (uint64_t i = start[k]; i < start[k + 1]; ++i) put(body[i]);
    }
    listing += '\n';
    if (n_raw) *n_raw = raw_lines;
    *needed = listing.size() + 1;
    if (out && capacity >= listing.size() + 1) memcpy(out, listing.c_str(), listing.size() + 1);
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

// ---- plain listing -> code -------------------------------------------------------------------

extern "C" int cubit_listing_assemble(cubit_ctx* ctx, const char* listing, const char* kernel, void* code,
                                      uint64_t capacity, uint64_t* needed, uint64_t* n_failed) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (!listing || !kernel || !needed) return fail(ctx, CUBIT_ERR_INVALID, "null argument");
    if (n_failed) *n_failed = 0;
    struct Line { uint32_t addr; bool raw; u128 word; std::string asm_text; bool has_sched; uint32_t sched; };
    std::vector<Line> lines;
    {
        // "/*<hex>*/" at the start of s (after blanks); returns the offset behind it or npos.
        auto addr_prefix = [](const std::string& s, uint32_t* addr) -> size_t {
            size_t i = 0;
            while (i < s.size() && isspace((unsigned char)s[i])) ++i;
            if (s.compare(i, 2, "/*") != 0) return std::string::npos;
            size_t k = i + 2;
            uint64_t v = 0;
            while (k < s.size() && (isdigit((unsigned char)s[k]) || (s[k] >= 'a' && s[k] <= 'f'))) {
                v = v * 16 + (uint64_t)(isdigit((unsigned char)s[k]) ? s[k] - '0' : s[k] - 'a' + 10);
                if (v > 0xFFFFFFFFull) v = 0;   // the reference falls back to address 0
                ++k;
            }
            if (k == i + 2 || s.compare(k, 2, "*/") != 0) return std::string::npos;
            k += 2;
            const size_t blanks = k;
            while (k < s.size() && isspace((unsigned char)s[k])) ++k;
            if (k == blanks) return std::string::npos;   // at least one blank follows
            *addr = (uint32_t)v;
            return k;
        };
        std::string current;
        const std::string text = listing;
        size_t pos = 0;
        while (pos <= text.size()) {
            size_t nl = text.find('\n', pos);
            if (nl == std::string::npos) nl = text.size();
            std::string line = text.substr(pos, nl - pos);
            pos = nl + 1;
            if (!line.empty() && line.back() == '\r') line.pop_back();
            size_t b = 0, e = line.size();
            while (b < e && isspace((unsigned char)line[b])) ++b;
            while (e > b && isspace((unsigned char)line[e - 1])) --e;
            const std::string t = line.substr(b, e - b);
            if (t.compare(0, 3, "// ") == 0 && t.find("/*") == std::string::npos) {
                size_t nb = 3, ne = t.size();
                while (nb < ne && isspace((unsigned char)t[nb])) ++nb;
                current = t.substr(nb);
                continue;
            }
            if (current != kernel) continue;
            uint32_t addr = 0;
            const size_t k = addr_prefix(t, &addr);
            if (k == std::string::npos) continue;
            // placeholder: /* ? 0x<hex> */
            {
                size_t q = k;
                if (t.compare(q, 2, "/*") == 0) {
                    q += 2;
                    while (q < t.size() && isspace((unsigned char)t[q])) ++q;
                    if (q < t.size() && t[q] == '?') {
                        ++q;
                        while (q < t.size() && isspace((unsigned char)t[q])) ++q;
                        if (t.compare(q, 2, "0x") == 0) {
                            size_t h = q + 2;
                            while (h < t.size() && isxdigit((unsigned char)t[h])) ++h;
                            size_t c = h;
                            while (c < t.size() && isspace((unsigned char)t[c])) ++c;
                            if (h > q + 2 && t.compare(c, 2, "*/") == 0) {
                                Line l{addr, true, 0, "", false, 0};
                                try {
                                    l.word = parse_hex_u128(t.substr(q + 2, h - q - 2));
                                    lines.push_back(l);
                                } catch (const std::exception&) {
                                    // wider than 128 bits: the reference drops the line as well
                                }
                                continue;
                            }
                        }
                    }
                }
            }
            const size_t semi = t.find(';', k);
            if (semi == std::string::npos) continue;
            size_t ae = semi;
            while (ae > k && isspace((unsigned char)t[ae - 1])) --ae;
            if (ae == k) continue;
            Line l{addr, false, 0, t.substr(k, ae - k), false, 0};
            const size_t sc = l.asm_text.find("/* @sched 0x");
            if (sc != std::string::npos) {
                const size_t vs = sc + 12;
                size_t ve = l.asm_text.find("*/", vs);
                if (ve == std::string::npos) { ve = l.asm_text.find(' ', vs); if (ve == std::string::npos) ve = l.asm_text.size(); }
                std::string hex = l.asm_text.substr(vs, ve - vs);
                while (!hex.empty() && isspace((unsigned char)hex.back())) hex.pop_back();
                char* end = nullptr;
                const unsigned long long v = strtoull(hex.c_str(), &end, 16);
                if (!hex.empty() && end && *end == 0) { l.has_sched = true; l.sched = (uint32_t)(v & 0x1FFFF); }
            }
            const size_t cut = l.asm_text.find("/* @sched");
            if (cut != std::string::npos) {
                l.asm_text = l.asm_text.substr(0, cut);
                while (!l.asm_text.empty() && isspace((unsigned char)l.asm_text.back())) l.asm_text.pop_back();
            }
            lines.push_back(l);
        }
    }
    uint64_t size = 0;
    for (const Line& l : lines) size = std::max<uint64_t>(size, (uint64_t)l.addr + 16);
    *needed = size;
    if (!code || capacity < size) return CUBIT_OK;
    memset(code, 0, size);

    // Lower on all host cores, encode in one batch, place every word at its address.
    const uint64_t total = lines.size();
    const unsigned parts = text_threads(total);
    std::vector<LoweredBatch> piece(parts);
    std::vector<std::vector<uint64_t>> piece_where(parts);
    std::vector<uint64_t> piece_failed(parts, 0);
    parallel_ranges(total, parts, [&](uint64_t b, uint64_t e, unsigned k) {
        static const char* const kNoWrite[] = {"EXIT", "BRA", "NOP", "RET", "BREAK", "CONT", "KILL", "STG", "STS", "ST", "STL",
                                               "STGX", "MEMBAR", "BAR", "BARRIER", "FENCE"};
        for (uint64_t i = b; i < e; ++i) {
            if (lines[i].raw) continue;
            try {
                TextInstruction insn = parse_sass(lines[i].asm_text, lines[i].addr);
                if (!lines[i].has_sched && insn.ctrl.write_bar == 7 && insn.ctrl.wait_mask == 0 && !insn.has_guard) {
                    bool no_write = false;
                    for (const char* op : kNoWrite) no_write |= insn.opcode == op;
                    if (!no_write && !insn.operands.empty() &&
                        (insn.operands[0].kind == OperandKind::Reg || insn.operands[0].kind == OperandKind::UReg))
                        insn.ctrl.write_bar = 1;
                }
                lower_one(ctx, insn, CUBIT_TEXT_ONE, &piece[k]);
                piece_where[k].push_back(i);
            } catch (const TextError&) {
                ++piece_failed[k];
            }
        }
    });
    LoweredBatch bt;
    std::vector<uint64_t> where;
    uint64_t failed = 0;
    for (unsigned k = 0; k < parts; ++k) {
        append_batch(&bt, piece[k]);
        where.insert(where.end(), piece_where[k].begin(), piece_where[k].end());
        failed += piece_failed[k];
    }
    const uint64_t m = where.size();
    std::vector<uint8_t> enc(16 * m);
    if (m) {
        std::vector<uint32_t> planes(8 * m);
        for (uint64_t i = 0; i < m; ++i)
            for (int s = 0; s < 8; ++s) planes[(uint64_t)s * m + i] = bt.slots[i * 8 + s];
        const int rc = cubit_encode_batch(ctx, bt.form.data(), planes.data(), bt.ctrl.data(), m, enc.data(), CUBIT_MEM_HOST, nullptr);
        if (rc) return rc;
    }
    uint8_t* out = (uint8_t*)code;
    for (uint64_t j = 0; j < m; ++j) {
        const Line& l = lines[where[j]];
        u128 w;
        memcpy(&w, enc.data() + j * 16, 16);
        w = (w & ~bt.clear[j]) | bt.set[j];
        if (l.has_sched) w = (w & ~((u128)0x1FFFF << 105)) | ((u128)l.sched << 105);
        memcpy(out + l.addr, &w, 16);
    }
    for (const Line& l : lines)
        if (l.raw) memcpy(out + l.addr, &l.word, 16);
    if (n_failed) *n_failed = failed;
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

// ---- cubin rewriting -------------------------------------------------------------------------

extern "C" int cubit_patch_elf(cubit_ctx* ctx, const cubit_elf* elf, void* out, uint64_t capacity, uint64_t* needed,
                               cubit_patch_stats* stats) try {
    if (!ctx) return CUBIT_ERR_INVALID;
    if (!elf || !needed) return fail(ctx, CUBIT_ERR_INVALID, "null argument");
    cubit_patch_stats st;
    memset(&st, 0, sizeof st);
    const uint32_t n_sec = (uint32_t)elf->text.size();
    std::vector<uint64_t> start(n_sec + 1, 0);
    int rc = cubit_decode_elf(ctx, elf, nullptr, n_sec, start.data(), 0, nullptr, nullptr, nullptr, nullptr, nullptr);
    if (rc) return rc;
    const uint64_t total = start.back();
    st.n_words = total;
    *needed = elf->len;
    if (!out || capacity < elf->len) { if (stats) *stats = st; return CUBIT_OK; }
    std::vector<uint16_t> form(total);
    std::vector<uint32_t> slots(8 * total), ctrl(total);
    std::vector<uint8_t> words(16 * total);
    if (total) {
        rc = cubit_decode_elf(ctx, elf, nullptr, n_sec, start.data(), total, form.data(), slots.data(), ctrl.data(),
                              words.data(), nullptr);
        if (rc) return rc;
    }
    // decode -> print -> parse -> lower on the host; what lowers is encoded in one batch.
    std::vector<std::string> text(total);
    std::vector<uint8_t> unknown(total, 0);
    std::vector<uint32_t> addr_of(total);
    for (uint32_t k = 0; k < n_sec; ++k)
        for (uint64_t i = start[k]; i < start[k + 1]; ++i) addr_of[i] = (uint32_t)((i - start[k]) * 16);
    parallel_ranges(total, text_threads(total), [&](uint64_t b0, uint64_t e0, unsigned) {
        for (uint64_t i = b0; i < e0; ++i) {
            unknown[i] = form[i] == 0xFFFFu;
            if (!unknown[i]) text[i] = print_word(ctx, words.data(), i, total, addr_of[i], form.data(), slots.data(), ctrl.data());
        }
    });
    LoweredBatch b;
    std::vector<uint64_t> where;
    lower_printed(ctx, text, unknown, addr_of, &b, &where);   // what does not parse or encode is kept as it is
    const uint64_t m = where.size();
    std::vector<uint8_t> enc(16 * m);
    if (m) {
        std::vector<uint32_t> planes(8 * m);
        for (uint64_t i = 0; i < m; ++i)
            for (int s = 0; s < 8; ++s) planes[(uint64_t)s * m + i] = b.slots[i * 8 + s];
        rc = cubit_encode_batch(ctx, b.form.data(), planes.data(), b.ctrl.data(), m, enc.data(), CUBIT_MEM_HOST, nullptr);
        if (rc) return rc;
    }
    memcpy(out, elf->bytes, elf->len);
    uint8_t* file = (uint8_t*)out;
    const u128 keep = ~((u128)0x1FFFF << 105);
    std::vector<uint64_t> file_off(total);
    for (uint32_t k = 0; k < n_sec; ++k)
        for (uint64_t i = start[k]; i < start[k + 1]; ++i) file_off[i] = elf->text[k].offset + (i - start[k]) * 16;
    for (uint64_t j = 0; j < m; ++j) {
        u128 e, w;
        memcpy(&e, enc.data() + j * 16, 16);
        memcpy(&w, words.data() + where[j] * 16, 16);
        e = (e & ~b.clear[j]) | b.set[j];
        if (((e ^ w) & keep) != 0) ++st.n_unfaithful;
        if ((uint64_t)e != (uint64_t)w) ++st.n_changed;
        const uint64_t lo = (uint64_t)e;
        memcpy(file + file_off[where[j]], &lo, 8);   // the high half stays the original's
    }
    st.n_reencoded = m;
    st.n_kept = total - m;
    if (stats) *stats = st;
    return CUBIT_OK;
} catch (...) {
    return translate_exception(ctx);
}

extern "C" int cubit_elf_patch_text(const cubit_elf* elf, uint32_t index, const void* code, uint64_t code_len, void* out,
                                    uint64_t capacity, uint64_t* needed) try {
    if (!elf || !needed || (code_len && !code)) return fail(nullptr, CUBIT_ERR_INVALID, "null argument");
    std::vector<uint8_t> file;
    try {
        file = elf_patch_text(elf->bytes, elf->len, index, (const uint8_t*)code, code_len);
    } catch (const std::exception& e) {
        return fail(nullptr, CUBIT_ERR_ELF, e.what());
    }
    *needed = file.size();
    if (out && capacity >= file.size()) memcpy(out, file.data(), file.size());
    return CUBIT_OK;
} catch (...) {
    return translate_exception(nullptr);
}
