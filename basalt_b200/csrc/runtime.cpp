// Launch runtime over the CUDA Driver API, resolved with dlopen so the library loads on a
// machine without a GPU. Stands in for crates/basalt-runtime/src/{dl,driver,context,module,
// ffi,error}.rs of the reference; see include/basalt_b200.h for the entry-by-entry mapping.
//
// Differences from the reference runtime, all deliberate:
//   * the device's primary context is retained instead of cuCtxCreate (driver.rs:143-159), so
//     device memory, streams and NCCL communicators are shared with the CUDA runtime in-process;
//   * launches take a stream and do not synchronise (module.rs:101-122 synchronises every launch);
//   * cuModuleLoadDataEx captures the JIT log (context.rs:43-61 uses cuModuleLoadData);
//   * kernels whose emitted PTX carries a `//!basalt.plan` line get their CUtensorMap
//     parameters built and appended at launch.
#include <cuda.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <thread>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/basalt_b200.h"
#include "../../include/basalt_b200_kernels.h"

namespace {

thread_local basalt_rt_error g_err;

int set_err(int kind, int code, const char* call, const std::string& msg) {
    memset(&g_err, 0, sizeof g_err);
    g_err.kind = kind;
    g_err.code = code;
    strncpy(g_err.call, call, sizeof g_err.call - 1);
    strncpy(g_err.message, msg.c_str(), sizeof g_err.message - 1);
    return kind;
}

struct Fns {
    CUresult (*cuInit)(unsigned);
    CUresult (*cuDeviceGetCount)(int*);
    CUresult (*cuDeviceGet)(CUdevice*, int);
    CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
    CUresult (*cuDevicePrimaryCtxRetain)(CUcontext*, CUdevice);
    CUresult (*cuDevicePrimaryCtxRelease)(CUdevice);
    CUresult (*cuCtxSetCurrent)(CUcontext);
    CUresult (*cuCtxSynchronize)();
    CUresult (*cuModuleLoadDataEx)(CUmodule*, const void*, unsigned, CUjit_option*, void**);
    CUresult (*cuModuleUnload)(CUmodule);
    CUresult (*cuModuleGetFunction)(CUfunction*, CUmodule, const char*);
    CUresult (*cuFuncSetAttribute)(CUfunction, CUfunction_attribute, int);
    CUresult (*cuLaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream, void**, void**);
    CUresult (*cuMemAlloc)(CUdeviceptr*, size_t);
    CUresult (*cuMemFree)(CUdeviceptr);
    CUresult (*cuMemcpyHtoD)(CUdeviceptr, const void*, size_t);
    CUresult (*cuMemcpyDtoH)(void*, CUdeviceptr, size_t);
    CUresult (*cuMemcpyHtoDAsync)(CUdeviceptr, const void*, size_t, CUstream);
    CUresult (*cuMemcpyDtoHAsync)(void*, CUdeviceptr, size_t, CUstream);
    CUresult (*cuPointerGetAttribute)(void*, CUpointer_attribute, CUdeviceptr);   // optional
    CUresult (*cuLaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**);   // optional
    CUresult (*cuMemAllocHost)(void**, size_t);
    CUresult (*cuMemFreeHost)(void*);
    CUresult (*cuStreamCreate)(CUstream*, unsigned);
    CUresult (*cuStreamDestroy)(CUstream);
    CUresult (*cuStreamSynchronize)(CUstream);
    CUresult (*cuEventCreate)(CUevent*, unsigned);
    CUresult (*cuEventDestroy)(CUevent);
    CUresult (*cuEventRecord)(CUevent, CUstream);
    CUresult (*cuEventSynchronize)(CUevent);
    CUresult (*cuEventElapsedTime)(float*, CUevent, CUevent);
    CUresult (*cuGetErrorString)(CUresult, const char**);
    CUresult (*cuOccupancyMaxActiveBlocksPerMultiprocessor)(int*, CUfunction, int, size_t);
    CUresult (*cuMemcpyDtoDAsync)(CUdeviceptr, CUdeviceptr, size_t, CUstream);
    CUresult (*cuStreamWaitEvent)(CUstream, CUevent, unsigned);
    CUresult (*cuIpcGetMemHandle)(CUipcMemHandle*, CUdeviceptr);
    CUresult (*cuIpcOpenMemHandle)(CUdeviceptr*, CUipcMemHandle, unsigned);
    CUresult (*cuIpcCloseMemHandle)(CUdeviceptr);
    CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
};

}  // namespace

struct basalt_rt_driver {
    void* lib = nullptr;
    Fns f{};
};
struct basalt_rt_ctx {
    basalt_rt_driver* drv = nullptr;
    CUdevice dev = 0;
    CUcontext ctx = nullptr;
    int sm_count = 0;
    // Device buffers kept between basalt_rt_cpu_launch calls, keyed by size: cuMemAlloc and
    // cuMemFree of a gigabyte cost more than the kernel they serve. Released with the context.
    std::multimap<size_t, CUdeviceptr> staging;
    // Workspace of kernels whose plan says `tail=`: two 128x128 f32 partial tiles per resident CTA (a stream
    // unit) and one ticket word per tile of a tail wave.  The kernels leave every ticket at zero.
    CUdeviceptr tail_partials = 0, tail_tickets = 0;
    // A launch that needs a larger workspace allocates a new one; the old one is kept until the context goes, because
    // launches already issued -- or captured in a CUDA graph -- still name it.
    std::vector<CUdeviceptr> tail_retired;
    unsigned tail_slots = 0;
    // Every launch of the context with stream units shares that workspace, so such launches are ordered one after
    // another: each records `tail_done` on its stream, and the next one on another stream first waits for it.
    CUevent tail_done = nullptr;
    CUstream tail_stream = nullptr;
    bool tail_pending = false;
    std::mutex mu;   // guards `staging` and the tail_* state: entry points may be called from several host threads
    // Lanes of the pageable-memory copy path of basalt_rt_cpu_launch (see staged_copy): per lane two pinned 4 MiB
    // buffers, a stream and two events.  Created on first use; one staged copy at a time (stage_mu).
    struct StageLane {
        void* pinned[2] = {nullptr, nullptr};
        CUstream stream = nullptr;
        CUevent done[2] = {nullptr, nullptr};
    };
    std::vector<StageLane> lanes;
    std::mutex stage_mu;
};
namespace {
struct TmapSpec {
    int param = 0;          // index of the pointer parameter the map is built over
    unsigned esz = 2;       // element bytes
    uint64_t inner = 0;     // elements per row
    uint64_t row_bytes = 0; // stride between rows
    unsigned box_inner = 0, box_outer = 0;
    unsigned swizzle = 0;   // bytes: 0, 32, 64, 128
    char outer_axis = 0;    // rows of the matrix: 'x' / 'y' = the caller's grid extent on that axis times outer_mult,
    uint64_t outer_mult = 0; //   0 = the constant outer_mult; both 0 = not known to the emitter (left wide open)
};
struct Plan {
    unsigned block[3] = {0, 0, 0};
    unsigned grid[3] = {0, 0, 0};
    unsigned smem = 0;
    unsigned nparams = 0;   // number of BIR parameters (tensor maps follow them)
    std::vector<TmapSpec> tmaps;
    std::string coarse;     // entry taking one more u64 parameter: the thread count the caller asked for
    unsigned per_thread = 0; // coarse entry: elements a thread handles in one trip of its loop (vector lanes x unroll)
    bool pdl = false;        // coarse entry: starts with griddepcontrol.wait, so it may be launched with programmatic stream serialisation
    bool status = false;    // the entry takes a u64 parameter: a device int32 set when a bounded wait gave up
    unsigned logical_block[3] = {0, 0, 0};   // block the caller must ask for when it differs from the block launched
    unsigned tail_k = 0;    // FFMA matmul with a streamed tail wave (K extent): the caller's 2-D grid is re-issued as a 1-D grid of
                            // whole tiles followed by stream units over the tail tiles; six trailing parameters (see basalt_rt_launch)
    std::string pair;       // persistent kernel only: the same kernel lowered for clusters of two CTAs that share a 2 x lgrid-wide,
                            // two-row tile; launched instead when the caller's grid is even in x and y
    unsigned lgrid = 0;     // persistent kernel: the caller's grid goes in two trailing u32 parameters; lgrid logical CTAs
                            // along x form one tile, and min(SM count, tiles) CTAs are launched
    unsigned pair_block = 0; // threads per CTA of the pair entry when they differ from block[0]
    int gather = -1;        // the kernel (its pair twin, for a persistent kernel) can also store its result behind peer base addresses:
                            // index of the output pointer parameter; two trailing parameters, a table of seven u64 and a u32 count
};
}  // namespace
struct basalt_rt_module {
    basalt_rt_ctx* ctx = nullptr;
    CUmodule mod = nullptr;
    std::map<std::string, Plan> plans;
};
struct basalt_rt_function {
    basalt_rt_module* mod = nullptr;
    CUfunction fn = nullptr;
    CUfunction coarse = nullptr;   // see Plan::coarse
    CUfunction pair = nullptr;     // see Plan::pair
    CUdeviceptr status = 0;        // see Plan::status
    bool use_pair = true;          // basalt_rt_function_tune: take the two-SM entry when the grid allows it
    bool tail_split = true;        //   work a sparse last wave off with stream units
    unsigned tail_rounds = 0;      //   rounds of stream units (0 = one, two with a gathering epilogue)
    unsigned coarse_waves = 0;     //   coarse entries: exactly this many resident waves (0 = one loop trip per thread)
    bool pdl = true;               //   coarse entries: launch with programmatic stream serialisation when the plan allows it
    bool has_plan = false;
    Plan plan;
};
struct basalt_rt_buffer {
    basalt_rt_ctx* ctx = nullptr;
    CUdeviceptr ptr = 0;
    size_t bytes = 0;
};
struct basalt_rt_comm {
    basalt_rt_ctx* ctx = nullptr;
    ncclComm_t comm = nullptr;
};
struct basalt_rt_peer_group {
    basalt_rt_ctx* ctx = nullptr;
    int nranks = 0, rank = 0;
    CUdeviceptr own = 0;                 // this rank's inbox; the status word sits kPeerStatusOffset bytes in
    uint64_t inbox[8] = {0};             // every rank's inbox as mapped on this device
    bool connected = false;
    uint32_t epoch = 0;
};

namespace {

// check() of the reference (driver.rs:65-90): a failing CUresult becomes DriverCallFailed with
// the driver's own message.
int check(const Fns& f, const char* call, CUresult rc) {
    if (rc == CUDA_SUCCESS) return 0;
    const char* msg = nullptr;
    std::string m;
    if (f.cuGetErrorString && f.cuGetErrorString(rc, &msg) == CUDA_SUCCESS && msg) m = msg;
    else m = "unknown CUDA error " + std::to_string((int)rc);
    return set_err(3, (int)rc, call, m);
}

template <class F>
bool resolve(void* lib, F* out, std::initializer_list<const char*> names) {
    for (const char* n : names) {
        void* p = dlsym(lib, n);
        if (p) { *out = reinterpret_cast<F>(p); return true; }
    }
    set_err(2, 0, "dlsym", std::string("CUDA driver symbol not found: ") + *names.begin());
    return false;
}

int make_current(basalt_rt_ctx* c) { return check(c->drv->f, "cuCtxSetCurrent", c->drv->f.cuCtxSetCurrent(c->ctx)); }

// ---- NCCL, resolved lazily ------------------------------------------------------------------
struct Nccl {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
};
Nccl* nccl() {
    static Nccl n;
    static bool tried = false, ok = false;
    if (!tried) {
        tried = true;
        n.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!n.lib) n.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (n.lib) {
            ok = resolve(n.lib, &n.GetUniqueId, {"ncclGetUniqueId"}) && resolve(n.lib, &n.CommInitRank, {"ncclCommInitRank"}) &&
                 resolve(n.lib, &n.CommDestroy, {"ncclCommDestroy"}) && resolve(n.lib, &n.AllReduce, {"ncclAllReduce"}) &&
                 resolve(n.lib, &n.AllGather, {"ncclAllGather"}) && resolve(n.lib, &n.GetErrorString, {"ncclGetErrorString"});
        }
    }
    if (!ok) { set_err(1, 0, "dlopen", "NCCL library not found (libnccl.so.2)"); return nullptr; }
    return &n;
}
int nccl_check(Nccl* n, const char* call, ncclResult_t rc) {
    if (rc == ncclSuccess) return 0;
    return set_err(5, (int)rc, call, n->GetErrorString(rc));
}

// Parses the `//!basalt.plan <kernel> key=value ...` lines of an emitted module.
void parse_plans(const char* ptx, std::map<std::string, Plan>* out) {
    std::istringstream in(ptx);
    std::string ln;
    while (std::getline(in, ln)) {
        if (ln.rfind("//!basalt.plan ", 0) != 0) continue;
        std::istringstream ls(ln.substr(15));
        std::string kernel, kv;
        ls >> kernel;
        Plan p;
        while (ls >> kv) {
            size_t eq = kv.find('=');
            if (eq == std::string::npos) continue;
            std::string k = kv.substr(0, eq), v = kv.substr(eq + 1);
            if (k == "block") sscanf(v.c_str(), "%u,%u,%u", &p.block[0], &p.block[1], &p.block[2]);
            else if (k == "grid") sscanf(v.c_str(), "%u,%u,%u", &p.grid[0], &p.grid[1], &p.grid[2]);
            else if (k == "smem") p.smem = (unsigned)strtoul(v.c_str(), nullptr, 10);
            else if (k == "params") p.nparams = (unsigned)strtoul(v.c_str(), nullptr, 10);
            else if (k == "coarse") p.coarse = v;
            else if (k == "per_thread") p.per_thread = (unsigned)strtoul(v.c_str(), nullptr, 10);
            else if (k == "pdl") p.pdl = v == "1";
            else if (k == "pair") p.pair = v;
            else if (k == "status") p.status = v != "0";
            else if (k == "logical_block") sscanf(v.c_str(), "%u,%u,%u", &p.logical_block[0], &p.logical_block[1], &p.logical_block[2]);
            else if (k == "lgrid") p.lgrid = (unsigned)strtoul(v.c_str(), nullptr, 10);
            else if (k == "tail") p.tail_k = (unsigned)strtoul(v.c_str(), nullptr, 10);
            else if (k == "gather") p.gather = (int)strtol(v.c_str(), nullptr, 10);
            else if (k == "pair_block") p.pair_block = (unsigned)strtoul(v.c_str(), nullptr, 10);
            else if (k == "tmap") {
                TmapSpec t;
                unsigned long long inner = 0, rowb = 0;
                char outer[32] = {0};
                if (sscanf(v.c_str(), "%d:%u:%llu:%llu:%u:%u:%u:%31s", &t.param, &t.esz, &inner, &rowb, &t.box_inner, &t.box_outer, &t.swizzle, outer) >= 7) {
                    t.inner = inner;
                    t.row_bytes = rowb;
                    if (outer[0] == 'x' || outer[0] == 'y') { t.outer_axis = outer[0]; t.outer_mult = strtoull(outer + 1, nullptr, 10); }
                    else if (outer[0]) t.outer_mult = strtoull(outer, nullptr, 10);
                    p.tmaps.push_back(t);
                }
            }
        }
        (*out)[kernel] = p;
    }
}

}  // namespace

extern "C" {

void basalt_rt_last_error(basalt_rt_error* out) {
    if (out) *out = g_err;
}

int basalt_rt_driver_load(basalt_rt_driver** out) {
    if (!out) return set_err(4, 0, "basalt_rt_driver_load", "null output pointer");
    *out = nullptr;
    void* lib = dlopen("libcuda.so.1", RTLD_NOW);
    if (!lib) lib = dlopen("libcuda.so", RTLD_NOW);
    if (!lib) {
        const char* e = dlerror();
        return set_err(1, 0, "dlopen", std::string("CUDA driver library not found: ") + (e ? e : "libcuda.so.1"));
    }
    auto* d = new basalt_rt_driver;
    d->lib = lib;
    Fns& f = d->f;
    bool ok = resolve(lib, &f.cuInit, {"cuInit"}) && resolve(lib, &f.cuDeviceGetCount, {"cuDeviceGetCount"}) &&
              resolve(lib, &f.cuDeviceGet, {"cuDeviceGet"}) && resolve(lib, &f.cuDeviceGetAttribute, {"cuDeviceGetAttribute"}) &&
              resolve(lib, &f.cuDevicePrimaryCtxRetain, {"cuDevicePrimaryCtxRetain"}) &&
              resolve(lib, &f.cuDevicePrimaryCtxRelease, {"cuDevicePrimaryCtxRelease_v2", "cuDevicePrimaryCtxRelease"}) &&
              resolve(lib, &f.cuCtxSetCurrent, {"cuCtxSetCurrent"}) && resolve(lib, &f.cuCtxSynchronize, {"cuCtxSynchronize"}) &&
              resolve(lib, &f.cuModuleLoadDataEx, {"cuModuleLoadDataEx"}) && resolve(lib, &f.cuModuleUnload, {"cuModuleUnload"}) &&
              resolve(lib, &f.cuModuleGetFunction, {"cuModuleGetFunction"}) && resolve(lib, &f.cuFuncSetAttribute, {"cuFuncSetAttribute"}) &&
              resolve(lib, &f.cuLaunchKernel, {"cuLaunchKernel"}) && resolve(lib, &f.cuMemAlloc, {"cuMemAlloc_v2", "cuMemAlloc"}) &&
              resolve(lib, &f.cuMemFree, {"cuMemFree_v2", "cuMemFree"}) && resolve(lib, &f.cuMemcpyHtoD, {"cuMemcpyHtoD_v2", "cuMemcpyHtoD"}) &&
              resolve(lib, &f.cuMemcpyDtoH, {"cuMemcpyDtoH_v2", "cuMemcpyDtoH"}) &&
              resolve(lib, &f.cuMemcpyHtoDAsync, {"cuMemcpyHtoDAsync_v2", "cuMemcpyHtoDAsync"}) &&
              resolve(lib, &f.cuMemcpyDtoHAsync, {"cuMemcpyDtoHAsync_v2", "cuMemcpyDtoHAsync"}) &&
              resolve(lib, &f.cuMemAllocHost, {"cuMemAllocHost_v2", "cuMemAllocHost"}) && resolve(lib, &f.cuMemFreeHost, {"cuMemFreeHost"}) &&
              resolve(lib, &f.cuStreamCreate, {"cuStreamCreate"}) && resolve(lib, &f.cuStreamDestroy, {"cuStreamDestroy_v2", "cuStreamDestroy"}) &&
              resolve(lib, &f.cuStreamSynchronize, {"cuStreamSynchronize"}) && resolve(lib, &f.cuEventCreate, {"cuEventCreate"}) &&
              resolve(lib, &f.cuEventDestroy, {"cuEventDestroy_v2", "cuEventDestroy"}) && resolve(lib, &f.cuEventRecord, {"cuEventRecord"}) &&
              resolve(lib, &f.cuEventSynchronize, {"cuEventSynchronize"}) && resolve(lib, &f.cuEventElapsedTime, {"cuEventElapsedTime"}) &&
              resolve(lib, &f.cuGetErrorString, {"cuGetErrorString", "cuGetErrorName"}) &&
              resolve(lib, &f.cuTensorMapEncodeTiled, {"cuTensorMapEncodeTiled"}) &&
              resolve(lib, &f.cuMemcpyDtoDAsync, {"cuMemcpyDtoDAsync_v2", "cuMemcpyDtoDAsync"}) &&
              resolve(lib, &f.cuStreamWaitEvent, {"cuStreamWaitEvent"}) &&
              resolve(lib, &f.cuIpcGetMemHandle, {"cuIpcGetMemHandle"}) &&
              resolve(lib, &f.cuIpcOpenMemHandle, {"cuIpcOpenMemHandle_v2", "cuIpcOpenMemHandle"}) &&
              resolve(lib, &f.cuIpcCloseMemHandle, {"cuIpcCloseMemHandle"}) &&
              resolve(lib, &f.cuOccupancyMaxActiveBlocksPerMultiprocessor, {"cuOccupancyMaxActiveBlocksPerMultiprocessor"});
    if (!ok) { dlclose(lib); delete d; return 2; }
    f.cuPointerGetAttribute = reinterpret_cast<decltype(f.cuPointerGetAttribute)>(dlsym(lib, "cuPointerGetAttribute"));   // optional
    f.cuLaunchKernelEx = reinterpret_cast<decltype(f.cuLaunchKernelEx)>(dlsym(lib, "cuLaunchKernelEx"));                  // optional
    int rc = check(f, "cuInit", f.cuInit(0));
    if (rc) { dlclose(lib); delete d; return rc; }
    *out = d;
    return 0;
}

void basalt_rt_driver_unload(basalt_rt_driver* drv) {
    if (!drv) return;
    // The library handle is kept open: unloading libcuda under a live CUDA runtime is not safe.
    delete drv;
}

int basalt_rt_device_count(basalt_rt_driver* drv, int* count) {
    if (!drv || !count) return set_err(4, 0, "basalt_rt_device_count", "null argument");
    return check(drv->f, "cuDeviceGetCount", drv->f.cuDeviceGetCount(count));
}

int basalt_rt_ctx_create(basalt_rt_driver* drv, int device_index, basalt_rt_ctx** out) {
    if (!drv || !out) return set_err(4, 0, "basalt_rt_ctx_create", "null argument");
    *out = nullptr;
    CUdevice dev;
    int rc = check(drv->f, "cuDeviceGet", drv->f.cuDeviceGet(&dev, device_index));
    if (rc) return rc;
    CUcontext ctx;
    rc = check(drv->f, "cuDevicePrimaryCtxRetain", drv->f.cuDevicePrimaryCtxRetain(&ctx, dev));
    if (rc) return rc;
    auto* c = new basalt_rt_ctx;
    c->drv = drv;
    c->dev = dev;
    c->ctx = ctx;
    rc = make_current(c);
    if (rc) { drv->f.cuDevicePrimaryCtxRelease(dev); delete c; return rc; }
    if (drv->f.cuDeviceGetAttribute(&c->sm_count, CU_DEVICE_ATTRIBUTE_MULTIPROCESSOR_COUNT, dev) != CUDA_SUCCESS || c->sm_count < 1) c->sm_count = 1;
    *out = c;
    return 0;
}

void basalt_rt_ctx_destroy(basalt_rt_ctx* ctx) {
    if (!ctx) return;
    for (auto& kv : ctx->staging) ctx->drv->f.cuMemFree(kv.second);
    for (auto& l : ctx->lanes) {
        for (int i = 0; i < 2; i++) {
            if (l.pinned[i]) ctx->drv->f.cuMemFreeHost(l.pinned[i]);
            if (l.done[i]) ctx->drv->f.cuEventDestroy(l.done[i]);
        }
        if (l.stream) ctx->drv->f.cuStreamDestroy(l.stream);
    }
    if (ctx->tail_partials) ctx->drv->f.cuMemFree(ctx->tail_partials);
    for (CUdeviceptr old : ctx->tail_retired) ctx->drv->f.cuMemFree(old);
    if (ctx->tail_tickets) ctx->drv->f.cuMemFree(ctx->tail_tickets);
    if (ctx->tail_done) ctx->drv->f.cuEventDestroy(ctx->tail_done);
    ctx->drv->f.cuDevicePrimaryCtxRelease(ctx->dev);
    delete ctx;
}

int basalt_rt_device_attr(basalt_rt_ctx* ctx, int attr, int* value) {
    if (!ctx || !value) return set_err(4, 0, "basalt_rt_device_attr", "null argument");
    return check(ctx->drv->f, "cuDeviceGetAttribute", ctx->drv->f.cuDeviceGetAttribute(value, (CUdevice_attribute)attr, ctx->dev));
}

int basalt_rt_module_load(basalt_rt_ctx* ctx, const char* ptx, basalt_rt_module** out) {
    if (!ctx || !ptx || !out) return set_err(4, 0, "basalt_rt_module_load", "null argument");
    *out = nullptr;
    int rc = make_current(ctx);
    if (rc) return rc;
    static thread_local char log[8192];
    log[0] = 0;
    CUjit_option opt[] = {CU_JIT_ERROR_LOG_BUFFER, CU_JIT_ERROR_LOG_BUFFER_SIZE_BYTES};
    void* val[] = {log, (void*)(uintptr_t)sizeof log};
    CUmodule mod;
    CUresult r = ctx->drv->f.cuModuleLoadDataEx(&mod, ptx, 2, opt, val);
    if (r != CUDA_SUCCESS) {
        check(ctx->drv->f, "cuModuleLoadData", r);
        if (log[0]) {
            std::string m = std::string(g_err.message) + ": " + log;
            strncpy(g_err.message, m.c_str(), sizeof g_err.message - 1);
        }
        return 3;
    }
    auto* m = new basalt_rt_module;
    m->ctx = ctx;
    m->mod = mod;
    parse_plans(ptx, &m->plans);
    *out = m;
    return 0;
}

void basalt_rt_module_unload(basalt_rt_module* mod) {
    if (!mod) return;
    mod->ctx->drv->f.cuModuleUnload(mod->mod);
    delete mod;
}

int basalt_rt_get_function(basalt_rt_module* mod, const char* name, basalt_rt_function** out) {
    if (!mod || !name || !out) return set_err(4, 0, "basalt_rt_get_function", "null argument");
    *out = nullptr;
    const Fns& f = mod->ctx->drv->f;
    CUfunction fn;
    int rc = check(f, "cuModuleGetFunction", f.cuModuleGetFunction(&fn, mod->mod, name));
    if (rc) return rc;
    auto* h = new basalt_rt_function;
    h->mod = mod;
    h->fn = fn;
    auto it = mod->plans.find(name);
    if (it != mod->plans.end()) {
        h->has_plan = true;
        h->plan = it->second;
        if (!h->plan.coarse.empty()) {
            rc = check(f, "cuModuleGetFunction", f.cuModuleGetFunction(&h->coarse, mod->mod, h->plan.coarse.c_str()));
            if (rc) { delete h; return rc; }
        }
        if (h->plan.status) {
            rc = check(f, "cuMemAlloc", f.cuMemAlloc(&h->status, 4));
            int32_t zero = 0;
            if (!rc) rc = check(f, "cuMemcpyHtoD", f.cuMemcpyHtoD(h->status, &zero, 4));
            if (rc) { delete h; return rc; }
        }
        if (!h->plan.pair.empty()) {
            rc = check(f, "cuModuleGetFunction", f.cuModuleGetFunction(&h->pair, mod->mod, h->plan.pair.c_str()));
            if (rc) { delete h; return rc; }
        }
        if (h->plan.smem > 48 * 1024) {
            rc = check(f, "cuFuncSetAttribute", f.cuFuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)h->plan.smem));
            if (!rc && h->pair) rc = check(f, "cuFuncSetAttribute", f.cuFuncSetAttribute(h->pair, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)h->plan.smem));
            if (rc) { delete h; return rc; }
        }
    }
    *out = h;
    return 0;
}

int basalt_rt_alloc(basalt_rt_ctx* ctx, size_t bytes, basalt_rt_buffer** out) {
    if (!ctx || !out) return set_err(4, 0, "basalt_rt_alloc", "null argument");
    *out = nullptr;
    int rc = make_current(ctx);
    if (rc) return rc;
    CUdeviceptr p = 0;
    rc = check(ctx->drv->f, "cuMemAlloc", ctx->drv->f.cuMemAlloc(&p, bytes ? bytes : 1));
    if (rc) return rc;
    auto* b = new basalt_rt_buffer;
    b->ctx = ctx;
    b->ptr = p;
    b->bytes = bytes;
    *out = b;
    return 0;
}

void basalt_rt_buffer_free(basalt_rt_buffer* buf) {
    if (!buf) return;
    buf->ctx->drv->f.cuMemFree(buf->ptr);
    delete buf;
}

uint64_t basalt_rt_buffer_ptr(const basalt_rt_buffer* buf) { return buf ? (uint64_t)buf->ptr : 0; }
size_t basalt_rt_buffer_size(const basalt_rt_buffer* buf) { return buf ? buf->bytes : 0; }

namespace {
constexpr size_t kStageMin = 2u << 20;     // smaller host buffers go through the driver's own pageable path
bool host_is_pinned(const Fns& f, const void* p);
int staged_copy(basalt_rt_ctx* ctx, CUdeviceptr dev, void* host, size_t bytes, bool to_device);
// A synchronous copy of a large pageable buffer: ordered after the work already in the NULL stream, like the
// driver's own synchronous copy, then moved by staged_copy.
int sync_staged(basalt_rt_ctx* ctx, CUdeviceptr dev, void* host, size_t bytes, bool to_device) {
    int rc = check(ctx->drv->f, "cuStreamSynchronize", ctx->drv->f.cuStreamSynchronize(nullptr));
    return rc ? rc : staged_copy(ctx, dev, host, bytes, to_device);
}
}  // namespace

int basalt_rt_copy_from_host(basalt_rt_buffer* buf, const void* host, size_t bytes, void* stream) {
    if (!buf || (!host && bytes)) return set_err(4, 0, "basalt_rt_copy_from_host", "null argument");
    if (bytes > buf->bytes) return set_err(4, 0, "cuMemcpyHtoD", "host slice of " + std::to_string(bytes) + " bytes exceeds the device buffer of " + std::to_string(buf->bytes));
    if (!bytes) return 0;
    const Fns& f = buf->ctx->drv->f;
    if (stream) return check(f, "cuMemcpyHtoDAsync", f.cuMemcpyHtoDAsync(buf->ptr, host, bytes, (CUstream)stream));
    if (bytes >= kStageMin && !host_is_pinned(f, host)) return sync_staged(buf->ctx, buf->ptr, const_cast<void*>(host), bytes, true);
    return check(f, "cuMemcpyHtoD", f.cuMemcpyHtoD(buf->ptr, host, bytes));
}

int basalt_rt_copy_to_host(const basalt_rt_buffer* buf, void* host, size_t bytes, void* stream) {
    if (!buf || (!host && bytes)) return set_err(4, 0, "basalt_rt_copy_to_host", "null argument");
    if (bytes > buf->bytes) return set_err(4, 0, "cuMemcpyDtoH", "host slice of " + std::to_string(bytes) + " bytes exceeds the device buffer of " + std::to_string(buf->bytes));
    if (!bytes) return 0;
    const Fns& f = buf->ctx->drv->f;
    if (stream) return check(f, "cuMemcpyDtoHAsync", f.cuMemcpyDtoHAsync(host, buf->ptr, bytes, (CUstream)stream));
    if (bytes >= kStageMin && !host_is_pinned(f, host)) return sync_staged(buf->ctx, buf->ptr, host, bytes, false);
    return check(f, "cuMemcpyDtoH", f.cuMemcpyDtoH(host, buf->ptr, bytes));
}

int basalt_rt_host_alloc(basalt_rt_ctx* ctx, size_t bytes, void** out) {
    if (!ctx || !out) return set_err(4, 0, "basalt_rt_host_alloc", "null argument");
    int rc = make_current(ctx);
    if (rc) return rc;
    return check(ctx->drv->f, "cuMemAllocHost", ctx->drv->f.cuMemAllocHost(out, bytes ? bytes : 1));
}
void basalt_rt_host_free(basalt_rt_ctx* ctx, void* p) {
    if (ctx && p) ctx->drv->f.cuMemFreeHost(p);
}

int basalt_rt_planned_geometry(basalt_rt_function* fn, void** params, uint32_t grid[3], uint32_t block[3], uint32_t* smem) {
    (void)params;
    if (!fn) return set_err(4, 0, "basalt_rt_planned_geometry", "null argument");
    for (int i = 0; i < 3; i++) {
        if (grid) grid[i] = fn->has_plan ? fn->plan.grid[i] : 0;
        if (block) block[i] = fn->has_plan ? fn->plan.block[i] : 0;
    }
    if (smem) *smem = fn->has_plan ? fn->plan.smem : 0;
    return 0;
}

// The schedule of an FFMA matmul whose plan says `tail=`: out = {full, per, units}.  Tiles [0, full) run whole, one CTA
// each.  The tiles of a last wave that does not fill the slots -- or a whole problem smaller than one wave -- are worked
// off by stream units: the tail tiles' K slabs (16 columns of A each) laid end to end, `per` = ceil(slabs / (slots x
// rounds)) to a unit, so every slot is busy for rounds x per / (K / 16) of a tile's time instead of one (256 tiles on 296
// slots: 0.87; 136 on 296: 0.46).  Against that stands the traffic of the partial sums (at most two 64 KB tiles written
// and read per unit, charged at 6 TB/s against a tile time of 0.17 us per K step); a gain below 3 % is not taken, and
// then full = tiles, per = units = 0.  A pure function of its arguments.
void basalt_rt_tail_plan(uint32_t tiles, uint32_t slots, uint32_t k_extent, uint32_t rounds, uint32_t out[3]) {
    out[0] = tiles;
    out[1] = out[2] = 0;
    if (slots == 0 || k_extent < 16) return;
    const uint64_t tail = tiles % slots, nkt = k_extent / 16;
    if (tail == 0 || tail * nkt >= (1ull << 31)) return;
    if (rounds < 1) rounds = 1;
    while (rounds > 1 && (tail * nkt) / ((uint64_t)slots * rounds) < 16) rounds--;   // at least 16 slabs to a unit
    const uint64_t want = (uint64_t)slots * rounds;
    const uint64_t pr = (tail * nkt + want - 1) / want;
    if (pr >= nkt) return;                                                            // no more units than tiles
    const uint64_t un = (tail * nkt + pr - 1) / pr;
    const double waves = (double)((un + slots - 1) / slots) * (double)pr / (double)nkt;
    const double cost = waves + (double)(2 * un) * 131072.0 / 6.0e6 / (0.17 * (double)k_extent);
    if (cost > 0.97) return;
    out[0] = tiles - (uint32_t)tail;
    out[1] = (uint32_t)pr;
    out[2] = (uint32_t)un;
}

namespace {
int launch_impl(basalt_rt_function* fn, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_mem_bytes, void* stream, void** params,
                const uint64_t* peer_out, int n_peers);

// One launch of `entry`.  When the function's plan says `pdl=1` -- the kernel's first instruction after its parameter
// loads is griddepcontrol.wait -- it goes out with programmatic stream serialisation: its CTAs may be set up while the
// kernel before it on the stream drains, and touch memory only once that kernel has completed, which hides the launch
// latency of back-to-back launches and keeps stream order.  An ordinary launch otherwise.
int launch_maybe_dependent(const Fns& f, const basalt_rt_function* fn, CUfunction entry, const uint32_t grid[3], const uint32_t block[3], uint32_t smem, void* stream,
                           void** params) {
    if (fn->pdl && fn->has_plan && fn->plan.pdl && f.cuLaunchKernelEx) {
        CUlaunchConfig cfg = {};
        cfg.gridDimX = grid[0]; cfg.gridDimY = grid[1]; cfg.gridDimZ = grid[2];
        cfg.blockDimX = block[0]; cfg.blockDimY = block[1]; cfg.blockDimZ = block[2];
        cfg.sharedMemBytes = smem;
        cfg.hStream = (CUstream)stream;
        CUlaunchAttribute attr = {};
        attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr.value.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        return check(f, "cuLaunchKernelEx", f.cuLaunchKernelEx(&cfg, entry, params, nullptr));
    }
    return check(f, "cuLaunchKernel", f.cuLaunchKernel(entry, grid[0], grid[1], grid[2], block[0], block[1], block[2], smem, (CUstream)stream, params, nullptr));
}
}
int basalt_rt_launch(basalt_rt_function* fn, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_mem_bytes, void* stream, void** params) {
    if (!fn || !grid || !block) return set_err(4, 0, "basalt_rt_launch", "null argument");
    return launch_impl(fn, grid, block, shared_mem_bytes, stream, params, nullptr, 0);
}

int basalt_rt_launch_gather(basalt_rt_function* fn, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_mem_bytes, void* stream, void** params,
                            const uint64_t* peer_out, int n_peers) {
    if (!fn || !grid || !block) return set_err(4, 0, "basalt_rt_launch_gather", "null argument");
    if (n_peers < 0 || n_peers > 7 || (n_peers && !peer_out)) return set_err(4, 0, "basalt_rt_launch_gather", "between 0 and 7 peer addresses");
    if (!fn->has_plan || fn->plan.gather < 0) return set_err(4, 0, "basalt_rt_launch_gather", "this kernel was not emitted with a gathering epilogue");
    for (int i = 0; i < n_peers; i++)
        if (!peer_out[i] || (peer_out[i] & 15)) return set_err(4, 0, "basalt_rt_launch_gather", "a peer address is null or not 16-byte aligned");
    return launch_impl(fn, grid, block, shared_mem_bytes, stream, params, peer_out, n_peers);
}

int basalt_rt_launch_gather_multicast(basalt_rt_function* fn, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_mem_bytes, void* stream, void** params,
                                      uint64_t multicast_out) {
    if (!fn || !grid || !block) return set_err(4, 0, "basalt_rt_launch_gather_multicast", "null argument");
    if (!fn->has_plan || fn->plan.gather < 0) return set_err(4, 0, "basalt_rt_launch_gather_multicast", "this kernel was not emitted with a gathering epilogue");
    if (!multicast_out || (multicast_out & 15)) return set_err(4, 0, "basalt_rt_launch_gather_multicast", "the multicast address is null or not 16-byte aligned");
    return launch_impl(fn, grid, block, shared_mem_bytes, stream, params, &multicast_out, -1);
}

namespace {
// n_peers = -1: peer_out[0] is the output's address in a multicast mapping of the whole group (the kernels see a count
// of one with bit 31 set).
int launch_impl(basalt_rt_function* fn, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_mem_bytes, void* stream, void** params,
                const uint64_t* peer_out, int n_peers) {
    const Fns& f = fn->mod->ctx->drv->f;
    uint64_t peer_table[7] = {0, 0, 0, 0, 0, 0, 0};
    uint32_t peer_count = (uint32_t)n_peers;
    if (n_peers < 0) {
        peer_table[0] = peer_out[0];
        peer_count = 0x80000001u;
        n_peers = 1;
    } else
        for (int i = 0; i < n_peers; i++) peer_table[i] = peer_out[i];
    if (fn->coarse && params && grid[1] == 1 && grid[2] == 1 && block[1] == 1 && block[2] == 1 && block[0] >= 32) {
        // One-element-per-thread kernel: the caller's launch names the logical threads.  They are run by CTAs whose
        // threads each make one trip of the vectorised loop (several 16-byte accesses in flight): many short CTAs
        // stream faster than one resident wave of long-running ones (vadd_i32 at 2^28: 6.9 against 6.1 TB/s), the
        // hardware scheduler evening out what the SMs and memory channels get.  Never fewer CTAs than would fill the
        // device when the work allows it, never more than the caller asked for.
        uint64_t logical = (uint64_t)grid[0] * block[0];
        int resident = 0;
        if (f.cuOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fn->coarse, (int)block[0], shared_mem_bytes) != CUDA_SUCCESS || resident < 1) resident = 1;
        uint64_t wave = (uint64_t)fn->mod->ctx->sm_count * (uint64_t)resident;
        uint64_t per_cta = (uint64_t)block[0] * (fn->plan.per_thread ? fn->plan.per_thread : 16);
        uint64_t want = (logical + per_cta - 1) / per_cta;
        if (fn->coarse_waves) want = wave * (uint64_t)fn->coarse_waves;   // basalt_rt_function_tune: a fixed number of waves
        if (want < wave) want = wave;
        uint32_t phys = grid[0] < want ? grid[0] : (uint32_t)want;
        std::vector<void*> all(params, params + fn->plan.nparams);
        all.push_back(&logical);
        const uint32_t one_d[3] = {phys, 1, 1}, blk[3] = {block[0], 1, 1};
        return launch_maybe_dependent(f, fn, fn->coarse, one_d, blk, shared_mem_bytes, stream, all.data());
    }
    if (fn->has_plan && fn->plan.tail_k) {
        // 128x128 tiles, one per logical CTA (grid x = tile column, y = tile row).  Whole tiles first,
        // then the tiles of a sparse last wave as stream units that keep every slot busy.
        const Plan& p = fn->plan;
        basalt_rt_ctx* ctx = fn->mod->ctx;
        const unsigned* want = p.logical_block[0] ? p.logical_block : p.block;
        if (block[0] != want[0] || block[1] != want[1] || block[2] != want[2])
            return set_err(4, 0, "cuLaunchKernel", "kernel was compiled for block (" + std::to_string(want[0]) + "," + std::to_string(want[1]) + "," + std::to_string(want[2]) + ")");
        if (grid[2] != 1) return set_err(4, 0, "cuLaunchKernel", "kernel was compiled for a two-dimensional grid");
        if (!params) return set_err(4, 0, "cuLaunchKernel", "kernel takes parameters");
        uint32_t lgx = grid[0], lgy = grid[1];
        const uint64_t tiles64 = (uint64_t)lgx * lgy;
        if (tiles64 == 0) return 0;
        if (tiles64 > 0x7fffffffull) return set_err(4, 0, "cuLaunchKernel", "grid too large");
        const uint32_t tiles = (uint32_t)tiles64;
        int resident = 0;
        if (f.cuOccupancyMaxActiveBlocksPerMultiprocessor(&resident, fn->fn, (int)p.block[0], p.smem) != CUDA_SUCCESS || resident < 1) resident = 1;
        const uint32_t slots = (uint32_t)ctx->sm_count * (uint32_t)resident;
        // With a gathering epilogue the units come in two rounds of one per slot (CTAs start in index order): the tiles
        // of the first round are complete, and on their way to the peers, while the second round computes; otherwise
        // every tile of the tail would finish, and leave, at the very end.
        uint32_t plan3[3] = {tiles, 0, 0};
        if (fn->tail_split) basalt_rt_tail_plan(tiles, slots, p.tail_k, fn->tail_rounds ? fn->tail_rounds : (n_peers > 0 ? 2u : 1u), plan3);
        uint32_t full = plan3[0], per = plan3[1], units = plan3[2];
        std::unique_lock<std::mutex> lock(ctx->mu, std::defer_lock);
        if (units) lock.lock();
        // two 64 KB partial tiles per unit, one ticket per tail tile (fewer than the units)
        const uint32_t need = std::max(2 * slots, 2 * units);
        if (units && ctx->tail_slots < need) {
            int rc = make_current(ctx);
            if (rc) return rc;
            if (ctx->tail_partials) {
                ctx->tail_retired.push_back(ctx->tail_partials);
                ctx->tail_retired.push_back(ctx->tail_tickets);
                ctx->tail_partials = ctx->tail_tickets = 0;
                ctx->tail_slots = 0;
            }
            rc = check(f, "cuMemAlloc", f.cuMemAlloc(&ctx->tail_partials, (size_t)need * 65536));
            if (rc) return rc;
            rc = check(f, "cuMemAlloc", f.cuMemAlloc(&ctx->tail_tickets, (size_t)need * 4));
            if (rc) { f.cuMemFree(ctx->tail_partials); ctx->tail_partials = 0; return rc; }
            std::vector<uint32_t> zeros(need, 0);
            rc = check(f, "cuMemcpyHtoD", f.cuMemcpyHtoD(ctx->tail_tickets, zeros.data(), (size_t)need * 4));
            if (rc) return rc;
            ctx->tail_slots = need;
        }
        std::vector<void*> all(params, params + p.nparams);
        uint64_t ws = (uint64_t)ctx->tail_partials, tk = (uint64_t)ctx->tail_tickets;
        all.push_back(&lgx);
        all.push_back(&lgy);
        all.push_back(&full);
        all.push_back(&per);
        all.push_back(&ws);
        all.push_back(&tk);
        if (p.gather >= 0) {
            all.push_back(peer_table);
            all.push_back(&peer_count);
        }
        if (units) {
            if (!ctx->tail_done) {
                int rc = check(f, "cuEventCreate", f.cuEventCreate(&ctx->tail_done, CU_EVENT_DISABLE_TIMING));
                if (rc) return rc;
            }
            if (ctx->tail_pending && ctx->tail_stream != (CUstream)stream) {
                int rc = check(f, "cuStreamWaitEvent", f.cuStreamWaitEvent((CUstream)stream, ctx->tail_done, 0));
                if (rc) return rc;
            }
        }
        int rc = check(f, "cuLaunchKernel", f.cuLaunchKernel(fn->fn, full + units, 1, 1, p.block[0], p.block[1], p.block[2], p.smem, (CUstream)stream, all.data(), nullptr));
        if (!rc && units) {
            rc = check(f, "cuEventRecord", f.cuEventRecord(ctx->tail_done, (CUstream)stream));
            ctx->tail_stream = (CUstream)stream;
            ctx->tail_pending = true;
        }
        return rc;
    }
    if (!fn->has_plan || fn->plan.tmaps.empty()) {
        if (fn->has_plan && fn->plan.block[0] && (block[0] != fn->plan.block[0] || block[1] != fn->plan.block[1] || block[2] != fn->plan.block[2]))
            return set_err(4, 0, "cuLaunchKernel", "kernel was compiled for block (" + std::to_string(fn->plan.block[0]) + "," + std::to_string(fn->plan.block[1]) + "," + std::to_string(fn->plan.block[2]) + ")");
        uint32_t sm = shared_mem_bytes ? shared_mem_bytes : (fn->has_plan ? fn->plan.smem : 0);
        return launch_maybe_dependent(f, fn, fn->fn, grid, block, sm, stream, params);
    }
    const Plan& p = fn->plan;
    const unsigned* want = p.logical_block[0] ? p.logical_block : p.block;
    if (block[0] != want[0] || block[1] != want[1] || block[2] != want[2])
        return set_err(4, 0, "cuLaunchKernel", "kernel was compiled for block (" + std::to_string(want[0]) + "," + std::to_string(want[1]) + "," + std::to_string(want[2]) + ")");
    if (!params) return set_err(4, 0, "cuLaunchKernel", "kernel takes parameters");
    std::vector<CUtensorMap> maps(p.tmaps.size());
    std::vector<void*> all(params, params + p.nparams);
    for (size_t i = 0; i < p.tmaps.size(); i++) {
        const TmapSpec& t = p.tmaps[i];
        if ((unsigned)t.param >= p.nparams) return set_err(4, 0, "cuTensorMapEncodeTiled", "plan names a parameter the kernel does not have");
        uint64_t base = *(uint64_t*)params[t.param];
        if (base & 15) return set_err(4, 0, "cuTensorMapEncodeTiled", "matrix base address must be 16-byte aligned");
        CUtensorMapDataType dt = t.esz == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : t.esz == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
        // The row count is not a kernel parameter: the plan derives it from the caller's grid (or names a
        // constant), so that a box that reaches past the matrix is clamped and zero-filled by the copy engine
        // instead of reading whatever lies behind the allocation; a kernel whose plan has no such field only
        // requests boxes inside its own matrix, and the extent is left wide open.
        cuuint64_t rows = (cuuint64_t)1 << 24;
        if (t.outer_axis == 'x') rows = (cuuint64_t)grid[0] * t.outer_mult;
        else if (t.outer_axis == 'y') rows = (cuuint64_t)grid[1] * t.outer_mult;
        else if (t.outer_mult) rows = t.outer_mult;
        if (rows == 0) return 0;
        cuuint64_t dims[2] = {t.inner, rows};
        cuuint64_t strides[1] = {t.row_bytes};
        cuuint32_t box[2] = {t.box_inner, t.box_outer};
        cuuint32_t estr[2] = {1, 1};
        CUtensorMapSwizzle sw = t.swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : t.swizzle == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : t.swizzle == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
        int rc = check(f, "cuTensorMapEncodeTiled",
                       f.cuTensorMapEncodeTiled(&maps[i], dt, 2, (void*)(uintptr_t)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
        if (rc) return rc;
        all.push_back(&maps[i]);
    }
    uint64_t status_ptr = (uint64_t)fn->status;
    if (p.status) all.push_back(&status_ptr);
    uint32_t sm = shared_mem_bytes ? shared_mem_bytes : p.smem;
    uint32_t g[3] = {grid[0], grid[1], grid[2]}, lgx = grid[0], lgy = grid[1];
    CUfunction entry = fn->fn;
    if (p.lgrid) {
        if (grid[2] != 1) return set_err(4, 0, "cuLaunchKernel", "kernel was compiled for a two-dimensional grid");
        uint64_t tiles = (uint64_t)((lgx + p.lgrid - 1) / p.lgrid) * lgy;
        uint64_t sms = (uint64_t)fn->mod->ctx->sm_count;
        g[0] = (uint32_t)(tiles < sms ? tiles : sms);
        g[1] = 1;
        if (fn->pair && fn->use_pair && p.lgrid == 2 && lgx % 2 == 0 && lgy % 2 == 0 && sms >= 2) {
            // clusters of two CTAs (the entry's own .reqnctapercluster), each walking tiles of 2 x 2 logical CTAs
            uint64_t pair_tiles = (uint64_t)(lgx / 2) * (lgy / 2);
            uint64_t pairs = pair_tiles < sms / 2 ? pair_tiles : sms / 2;
            g[0] = (uint32_t)(2 * pairs);
            entry = fn->pair;
        }
        if (g[0] == 0) return 0;
        all.push_back(&lgx);
        all.push_back(&lgy);
        if (entry == fn->pair && p.gather >= 0) {
            all.push_back(peer_table);
            all.push_back(&peer_count);
        }
    }
    if (n_peers && !(entry == fn->pair && p.gather >= 0))
        return set_err(4, 0, "basalt_rt_launch_gather", "the gathering epilogue is in the two-SM entry: the grid must be even in x and y");
    const unsigned threads = entry == fn->pair && p.pair_block ? p.pair_block : p.block[0];
    return check(f, "cuLaunchKernel", f.cuLaunchKernel(entry, g[0], g[1], g[2], threads, p.block[1], p.block[2], sm, (CUstream)stream, all.data(), nullptr));
}
}  // namespace

int basalt_rt_function_tune(basalt_rt_function* fn, const char* key, int value) {
    if (!fn || !key) return set_err(4, 0, "basalt_rt_function_tune", "null argument");
    const std::string k = key;
    if (k == "pair") fn->use_pair = value != 0;
    else if (k == "tail_split") fn->tail_split = value != 0;
    else if (k == "tail_rounds") fn->tail_rounds = value < 0 ? 0u : value > 8 ? 8u : (unsigned)value;
    else if (k == "coarse_waves") fn->coarse_waves = value > 0 ? (unsigned)value : 0;
    else if (k == "pdl") fn->pdl = value != 0;
    else return set_err(4, 0, "basalt_rt_function_tune", "unknown key: " + k);
    return 0;
}

int basalt_rt_occupancy(basalt_rt_function* fn, uint32_t block_threads, uint32_t shared_mem_bytes, int* ctas_per_sm, int* sm_count) {
    if (!fn || !ctas_per_sm) return set_err(4, 0, "basalt_rt_occupancy", "null argument");
    const Fns& f = fn->mod->ctx->drv->f;
    if (sm_count) *sm_count = fn->mod->ctx->sm_count;
    uint32_t sm = shared_mem_bytes ? shared_mem_bytes : (fn->has_plan ? fn->plan.smem : 0);
    return check(f, "cuOccupancyMaxActiveBlocksPerMultiprocessor", f.cuOccupancyMaxActiveBlocksPerMultiprocessor(ctas_per_sm, fn->fn, (int)block_threads, sm));
}

int basalt_rt_kernel_status(basalt_rt_function* fn, int32_t* out) {
    if (!fn || !out) return set_err(4, 0, "basalt_rt_kernel_status", "null argument");
    *out = 0;
    if (!fn->status) return 0;
    const Fns& f = fn->mod->ctx->drv->f;
    return check(f, "cuMemcpyDtoH", f.cuMemcpyDtoH(out, fn->status, 4));
}

int basalt_rt_ctx_sync(basalt_rt_ctx* ctx) {
    if (!ctx) return set_err(4, 0, "basalt_rt_ctx_sync", "null argument");
    int rc = make_current(ctx);
    if (rc) return rc;
    return check(ctx->drv->f, "cuCtxSynchronize", ctx->drv->f.cuCtxSynchronize());
}

int basalt_rt_stream_create(basalt_rt_ctx* ctx, void** out) {
    if (!ctx || !out) return set_err(4, 0, "basalt_rt_stream_create", "null argument");
    int rc = make_current(ctx);
    if (rc) return rc;
    return check(ctx->drv->f, "cuStreamCreate", ctx->drv->f.cuStreamCreate((CUstream*)out, CU_STREAM_NON_BLOCKING));
}
int basalt_rt_stream_destroy(basalt_rt_ctx* ctx, void* s) { return ctx ? check(ctx->drv->f, "cuStreamDestroy", ctx->drv->f.cuStreamDestroy((CUstream)s)) : 4; }
int basalt_rt_stream_sync(basalt_rt_ctx* ctx, void* s) { return ctx ? check(ctx->drv->f, "cuStreamSynchronize", ctx->drv->f.cuStreamSynchronize((CUstream)s)) : 4; }
int basalt_rt_event_create(basalt_rt_ctx* ctx, void** out) {
    if (!ctx || !out) return set_err(4, 0, "basalt_rt_event_create", "null argument");
    int rc = make_current(ctx);
    if (rc) return rc;
    return check(ctx->drv->f, "cuEventCreate", ctx->drv->f.cuEventCreate((CUevent*)out, CU_EVENT_DEFAULT));
}
int basalt_rt_event_destroy(basalt_rt_ctx* ctx, void* e) { return ctx ? check(ctx->drv->f, "cuEventDestroy", ctx->drv->f.cuEventDestroy((CUevent)e)) : 4; }
int basalt_rt_event_record(basalt_rt_ctx* ctx, void* e, void* s) { return ctx ? check(ctx->drv->f, "cuEventRecord", ctx->drv->f.cuEventRecord((CUevent)e, (CUstream)s)) : 4; }
int basalt_rt_event_sync(basalt_rt_ctx* ctx, void* e) { return ctx ? check(ctx->drv->f, "cuEventSynchronize", ctx->drv->f.cuEventSynchronize((CUevent)e)) : 4; }
int basalt_rt_event_elapsed_ms(basalt_rt_ctx* ctx, void* a, void* b, float* ms) {
    return ctx ? check(ctx->drv->f, "cuEventElapsedTime", ctx->drv->f.cuEventElapsedTime(ms, (CUevent)a, (CUevent)b)) : 4;
}

namespace {
constexpr size_t kStageChunk = 4u << 20;   // bytes per pinned buffer
constexpr int kStageLanesMax = 8;          // host threads that copy, each with its own stream: half the CPUs, 2 to 8

// True when the driver knows `p` as page-locked host memory (cuMemAllocHost, cuMemHostRegister): copies from it run at
// PCIe speed already.  Pageable memory is unknown to the driver (the query fails).
bool host_is_pinned(const Fns& f, const void* p) {
    if (!f.cuPointerGetAttribute) return true;
    unsigned type = 0;
    return f.cuPointerGetAttribute(&type, CU_POINTER_ATTRIBUTE_MEMORY_TYPE, (CUdeviceptr)(uintptr_t)p) == CUDA_SUCCESS && type == (unsigned)CU_MEMORYTYPE_HOST;
}

// Copy between pageable host memory and the device: the callers of the reference's CPU launch ABI pass malloc'd
// buffers (examples/cpu_launch_*.c), which the driver moves at about 11 GB/s on these hosts through its own staging
// buffer.  Here up to eight host threads take the 4 MiB chunks in turn, each copies its chunk into (out of) one of its two pinned
// buffers and hands it to the copy engine on its own stream, so that the memcpy of one chunk overlaps the DMA of
// others and several cores share the memcpy (1 GiB up: 11 GB/s through the driver's path, 39 with four threads, 43.5 with
// eight; 55 from page-locked memory).
int staged_copy(basalt_rt_ctx* ctx, CUdeviceptr dev, void* host, size_t bytes, bool to_device) {
    const Fns& f = ctx->drv->f;
    std::lock_guard<std::mutex> g(ctx->stage_mu);
    if (ctx->lanes.empty()) {
        const unsigned cpus = std::thread::hardware_concurrency();
        std::vector<basalt_rt_ctx::StageLane> lanes((size_t)std::min(kStageLanesMax, std::max(2, (int)cpus / 2)));
        bool ok = true;
        for (auto& l : lanes) {
            ok = ok && f.cuStreamCreate(&l.stream, CU_STREAM_NON_BLOCKING) == CUDA_SUCCESS;
            for (int i = 0; i < 2; i++)
                ok = ok && f.cuMemAllocHost(&l.pinned[i], kStageChunk) == CUDA_SUCCESS && f.cuEventCreate(&l.done[i], CU_EVENT_DISABLE_TIMING) == CUDA_SUCCESS;
        }
        if (!ok) {   // no pinned memory to be had: the driver's path still works
            for (auto& l : lanes) {
                for (int i = 0; i < 2; i++) {
                    if (l.pinned[i]) f.cuMemFreeHost(l.pinned[i]);
                    if (l.done[i]) f.cuEventDestroy(l.done[i]);
                }
                if (l.stream) f.cuStreamDestroy(l.stream);
            }
            return to_device ? check(f, "cuMemcpyHtoD", f.cuMemcpyHtoD(dev, host, bytes)) : check(f, "cuMemcpyDtoH", f.cuMemcpyDtoH(host, dev, bytes));
        }
        ctx->lanes = std::move(lanes);
    }
    const size_t chunk = bytes >= (32u << 20) ? kStageChunk : (1u << 20);   // small buffers in 1 MiB pieces, so that several threads share them
    const size_t nchunks = (bytes + chunk - 1) / chunk;
    const int nlanes = (int)std::min<size_t>(ctx->lanes.size(), nchunks);
    std::atomic<int> failed{0};
    auto lane_work = [&](int li) {
        if (f.cuCtxSetCurrent(ctx->ctx) != CUDA_SUCCESS) { failed = 1; return; }
        auto& l = ctx->lanes[li];
        char* h = static_cast<char*>(host);
        auto span = [&](size_t c, size_t* off, size_t* len) { *off = c * chunk; *len = std::min(chunk, bytes - *off); };
        size_t off, len;
        if (to_device) {
            int k = 0;
            for (size_t c = (size_t)li; c < nchunks && !failed; c += nlanes, k++) {
                const int s = k & 1;
                span(c, &off, &len);
                if (k >= 2 && f.cuEventSynchronize(l.done[s]) != CUDA_SUCCESS) { failed = 1; break; }   // the DMA that last read this buffer
                memcpy(l.pinned[s], h + off, len);
                if (f.cuMemcpyHtoDAsync(dev + off, l.pinned[s], len, l.stream) != CUDA_SUCCESS || f.cuEventRecord(l.done[s], l.stream) != CUDA_SUCCESS) { failed = 1; break; }
            }
        } else {
            auto fetch = [&](size_t c, int s) {
                span(c, &off, &len);
                if (f.cuMemcpyDtoHAsync(l.pinned[s], dev + off, len, l.stream) != CUDA_SUCCESS || f.cuEventRecord(l.done[s], l.stream) != CUDA_SUCCESS) failed = 1;
            };
            int k = 0;
            if ((size_t)li < nchunks) fetch((size_t)li, 0);
            for (size_t c = (size_t)li; c < nchunks && !failed; c += nlanes, k++) {
                const int s = k & 1;
                if (c + nlanes < nchunks) fetch(c + nlanes, s ^ 1);   // the next chunk lands while this one is copied out
                if (failed || f.cuEventSynchronize(l.done[s]) != CUDA_SUCCESS) { failed = 1; break; }
                span(c, &off, &len);
                memcpy(h + off, l.pinned[s], len);
            }
        }
        if (f.cuStreamSynchronize(l.stream) != CUDA_SUCCESS) failed = 1;
    };
    std::vector<std::thread> helpers;
    for (int li = 1; li < nlanes; li++) helpers.emplace_back(lane_work, li);
    lane_work(0);
    for (auto& t : helpers) t.join();
    if (failed) return set_err(3, 0, to_device ? "cuMemcpyHtoDAsync" : "cuMemcpyDtoHAsync", "a staged copy between pageable host memory and the device failed");
    return 0;
}
}  // namespace

int basalt_rt_cpu_launch(basalt_rt_ctx* ctx, basalt_rt_function* fn, const basalt_rt_arg* args, int nargs, int64_t nthreads, uint32_t block) {
    if (!ctx || !fn || (nargs && !args) || nthreads < 0 || block == 0) return set_err(4, 0, "basalt_rt_cpu_launch", "bad argument");
    const Fns& f = ctx->drv->f;
    int rc = make_current(ctx);
    if (rc) return rc;
    std::vector<std::pair<size_t, CUdeviceptr>> held(nargs, {0, 0});
    std::vector<uint64_t> dptrs(nargs, 0);
    std::vector<void*> params(nargs, nullptr);
    auto release = [&]() {
        std::lock_guard<std::mutex> g(ctx->mu);
        for (auto& h : held) if (h.second) ctx->staging.insert(h);
    };
    for (int i = 0; i < nargs && !rc; i++) {
        const basalt_rt_arg& a = args[i];
        if (a.kind >= 4) {
            size_t bytes = a.bytes ? a.bytes : 1;
            CUdeviceptr p = 0;
            {
                std::lock_guard<std::mutex> g(ctx->mu);
                auto it = ctx->staging.find(bytes);
                if (it != ctx->staging.end()) { p = it->second; ctx->staging.erase(it); }
            }
            if (!p) rc = check(f, "cuMemAlloc", f.cuMemAlloc(&p, bytes));
            if (rc) break;
            held[i] = {bytes, p};
            // written-only buffers are uploaded too: the kernel may leave part of them untouched
            if (a.bytes) {
                if (a.bytes >= kStageMin && !host_is_pinned(f, a.host)) rc = staged_copy(ctx, p, a.host, a.bytes, true);
                else rc = check(f, "cuMemcpyHtoD", f.cuMemcpyHtoD(p, a.host, a.bytes));
            }
            dptrs[i] = (uint64_t)p;
            params[i] = &dptrs[i];
        } else params[i] = (void*)&a.value;
    }
    if (!rc && nthreads > 0) {
        uint32_t grid[3] = {(uint32_t)((nthreads + block - 1) / block), 1, 1};
        uint32_t blk[3] = {(uint32_t)(nthreads < (int64_t)block ? nthreads : block), 1, 1};
        rc = basalt_rt_launch(fn, grid, blk, 0, nullptr, params.data());
        if (!rc) rc = basalt_rt_ctx_sync(ctx);
    }
    for (int i = 0; i < nargs && !rc; i++)
        if ((args[i].kind == 5 || args[i].kind == 6) && args[i].bytes) {
            if (args[i].bytes >= kStageMin && !host_is_pinned(f, args[i].host)) rc = staged_copy(ctx, (CUdeviceptr)dptrs[i], args[i].host, args[i].bytes, false);
            else rc = check(f, "cuMemcpyDtoH", f.cuMemcpyDtoH(args[i].host, (CUdeviceptr)dptrs[i], args[i].bytes));
        }
    release();
    return rc;
}

void basalt_rt_shard_range(uint64_t total, int nranks, int rank, uint64_t align, uint64_t* begin, uint64_t* end) {
    if (align == 0) align = 1;
    if (nranks < 1) nranks = 1;
    uint64_t units = (total + align - 1) / align;   // aligned chunks, the last possibly partial
    uint64_t per = units / (uint64_t)nranks, extra = units % (uint64_t)nranks;
    uint64_t r = (uint64_t)rank;
    uint64_t b = r * per + (r < extra ? r : extra), e = b + per + (r < extra ? 1 : 0);
    b *= align;
    e *= align;
    if (b > total) b = total;
    if (e > total) e = total;
    if (begin) *begin = b;
    if (end) *end = e;
}

int basalt_rt_comm_unique_id(char id_out[128]) {
    Nccl* n = nccl();
    if (!n) return 1;
    ncclUniqueId id;
    int rc = nccl_check(n, "ncclGetUniqueId", n->GetUniqueId(&id));
    if (rc) return rc;
    static_assert(sizeof id == 128, "ncclUniqueId is 128 bytes");
    memcpy(id_out, &id, 128);
    return 0;
}

int basalt_rt_comm_init(basalt_rt_ctx* ctx, const char id[128], int nranks, int rank, basalt_rt_comm** out) {
    if (!ctx || !id || !out) return set_err(4, 0, "basalt_rt_comm_init", "null argument");
    *out = nullptr;
    Nccl* n = nccl();
    if (!n) return 1;
    int rc = make_current(ctx);
    if (rc) return rc;
    ncclUniqueId uid;
    memcpy(&uid, id, 128);
    ncclComm_t c;
    rc = nccl_check(n, "ncclCommInitRank", n->CommInitRank(&c, nranks, uid, rank));
    if (rc) return rc;
    auto* h = new basalt_rt_comm;
    h->ctx = ctx;
    h->comm = c;
    *out = h;
    return 0;
}

void basalt_rt_comm_destroy(basalt_rt_comm* comm) {
    if (!comm) return;
    if (Nccl* n = nccl()) n->CommDestroy(comm->comm);
    delete comm;
}

int basalt_rt_allreduce_max_i32(basalt_rt_comm* comm, uint64_t send, uint64_t recv, size_t count, void* stream) {
    Nccl* n = nccl();
    if (!n || !comm) return set_err(4, 0, "basalt_rt_allreduce_max_i32", "no communicator");
    return nccl_check(n, "ncclAllReduce", n->AllReduce((const void*)(uintptr_t)send, (void*)(uintptr_t)recv, count, ncclInt32, ncclMax, comm->comm, (cudaStream_t)stream));
}

int basalt_rt_allgather(basalt_rt_comm* comm, uint64_t send, uint64_t recv, size_t bytes_per_rank, void* stream) {
    Nccl* n = nccl();
    if (!n || !comm) return set_err(4, 0, "basalt_rt_allgather", "no communicator");
    return nccl_check(n, "ncclAllGather", n->AllGather((const void*)(uintptr_t)send, (void*)(uintptr_t)recv, bytes_per_rank, ncclUint8, comm->comm, (cudaStream_t)stream));
}

// ---- peer mappings of whole buffers, device-to-device copies, cross-stream ordering --------------
int basalt_rt_ipc_export(const basalt_rt_buffer* buf, unsigned char handle_out[64]) {
    if (!buf || !handle_out) return set_err(4, 0, "basalt_rt_ipc_export", "null argument");
    int rc = make_current(buf->ctx);
    if (rc) return rc;
    CUipcMemHandle h;
    rc = check(buf->ctx->drv->f, "cuIpcGetMemHandle", buf->ctx->drv->f.cuIpcGetMemHandle(&h, buf->ptr));
    if (rc) return rc;
    memcpy(handle_out, &h, 64);
    return 0;
}

int basalt_rt_ipc_open(basalt_rt_ctx* ctx, const unsigned char handle[64], uint64_t* ptr_out) {
    if (!ctx || !handle || !ptr_out) return set_err(4, 0, "basalt_rt_ipc_open", "null argument");
    int rc = make_current(ctx);
    if (rc) return rc;
    CUipcMemHandle h;
    memcpy(&h, handle, 64);
    CUdeviceptr p = 0;
    rc = check(ctx->drv->f, "cuIpcOpenMemHandle", ctx->drv->f.cuIpcOpenMemHandle(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS));
    if (rc) return rc;
    *ptr_out = (uint64_t)p;
    return 0;
}

int basalt_rt_ipc_close(basalt_rt_ctx* ctx, uint64_t ptr) {
    if (!ctx || !ptr) return set_err(4, 0, "basalt_rt_ipc_close", "null argument");
    int rc = make_current(ctx);
    if (rc) return rc;
    return check(ctx->drv->f, "cuIpcCloseMemHandle", ctx->drv->f.cuIpcCloseMemHandle((CUdeviceptr)ptr));
}

int basalt_rt_copy_device_async(basalt_rt_ctx* ctx, uint64_t dst, uint64_t src, size_t bytes, void* stream) {
    if (!ctx || ((!dst || !src) && bytes)) return set_err(4, 0, "basalt_rt_copy_device_async", "null argument");
    if (!bytes) return 0;
    return check(ctx->drv->f, "cuMemcpyDtoDAsync", ctx->drv->f.cuMemcpyDtoDAsync((CUdeviceptr)dst, (CUdeviceptr)src, bytes, (CUstream)stream));
}

int basalt_rt_stream_wait_event(basalt_rt_ctx* ctx, void* stream, void* event) {
    if (!ctx || !event) return set_err(4, 0, "basalt_rt_stream_wait_event", "null argument");
    return check(ctx->drv->f, "cuStreamWaitEvent", ctx->drv->f.cuStreamWaitEvent((CUstream)stream, (CUevent)event, 0));
}

// ---- peer-memory exchange group ---------------------------------------------------------------
static const size_t kPeerInboxBytes = 2u << 20;      // its own allocation granule, so the IPC mapping covers nothing else
static const size_t kPeerStatusOffset = 4096;
static const size_t kPeerTicketOffset = 4096 + 64;    // ticket of the fused reduction + exchange kernel, starts at 0
static const size_t kPeerPartialOffset = 4096 + 128;  // its running maximum, starts at INT32_MIN
static const uint64_t kPeerTimeoutNs = 2000000000ull;

int basalt_rt_peer_group_create(basalt_rt_ctx* ctx, int nranks, int rank, basalt_rt_peer_group** out) {
    if (!ctx || !out) return set_err(4, 0, "basalt_rt_peer_group_create", "null argument");
    *out = nullptr;
    if (nranks < 1 || nranks > 8 || rank < 0 || rank >= nranks) return set_err(4, 0, "basalt_rt_peer_group_create", "rank or world size out of range (at most 8 ranks)");
    int rc = make_current(ctx);
    if (rc) return rc;
    const Fns& f = ctx->drv->f;
    CUdeviceptr p = 0;
    rc = check(f, "cuMemAlloc", f.cuMemAlloc(&p, kPeerInboxBytes));
    if (rc) return rc;
    std::vector<unsigned char> zeros(8192, 0);
    const int32_t lowest = INT32_MIN;
    memcpy(zeros.data() + kPeerPartialOffset, &lowest, 4);
    rc = check(f, "cuMemcpyHtoD", f.cuMemcpyHtoD(p, zeros.data(), zeros.size()));
    if (rc) { f.cuMemFree(p); return rc; }
    auto* g = new basalt_rt_peer_group;
    g->ctx = ctx;
    g->nranks = nranks;
    g->rank = rank;
    g->own = p;
    g->inbox[rank] = (uint64_t)p;
    g->connected = nranks == 1;
    *out = g;
    return 0;
}

int basalt_rt_peer_group_handle(basalt_rt_peer_group* g, unsigned char handle_out[64]) {
    if (!g || !handle_out) return set_err(4, 0, "basalt_rt_peer_group_handle", "null argument");
    static_assert(sizeof(CUipcMemHandle) == 64, "CUDA IPC handles are 64 bytes");
    int rc = make_current(g->ctx);
    if (rc) return rc;
    CUipcMemHandle h;
    rc = check(g->ctx->drv->f, "cuIpcGetMemHandle", g->ctx->drv->f.cuIpcGetMemHandle(&h, g->own));
    if (rc) return rc;
    memcpy(handle_out, &h, 64);
    return 0;
}

int basalt_rt_peer_group_connect(basalt_rt_peer_group* g, const unsigned char* handles, size_t nbytes) {
    if (!g || !handles) return set_err(4, 0, "basalt_rt_peer_group_connect", "null argument");
    if (nbytes != (size_t)g->nranks * 64) return set_err(4, 0, "basalt_rt_peer_group_connect", "expected one 64-byte handle per rank");
    if (g->connected) return set_err(4, 0, "basalt_rt_peer_group_connect", "already connected");
    int rc = make_current(g->ctx);
    if (rc) return rc;
    const Fns& f = g->ctx->drv->f;
    for (int r = 0; r < g->nranks; r++) {
        if (r == g->rank) continue;
        CUipcMemHandle h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        CUdeviceptr p = 0;
        rc = check(f, "cuIpcOpenMemHandle", f.cuIpcOpenMemHandle(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS));
        if (rc) {
            for (int q = 0; q < r; q++) if (q != g->rank && g->inbox[q]) { f.cuIpcCloseMemHandle((CUdeviceptr)g->inbox[q]); g->inbox[q] = 0; }
            return rc;
        }
        g->inbox[r] = (uint64_t)p;
    }
    g->connected = true;
    return 0;
}

int basalt_rt_peer_allreduce_max_i32(basalt_rt_peer_group* g, uint64_t partial, uint64_t result, int reset, int32_t reset_value, void* stream) {
    if (!g || !partial || !result) return set_err(4, 0, "basalt_rt_peer_allreduce_max_i32", "null argument");
    if (!g->connected) return set_err(4, 0, "basalt_rt_peer_allreduce_max_i32", "the group is not connected");
    int rc = make_current(g->ctx);
    if (rc) return rc;
    if (++g->epoch == 0) g->epoch = 1;
    int krc = basalt_k_peer_allreduce_max_i32(g->inbox, g->nranks, g->rank, g->epoch, (int32_t*)(uintptr_t)partial, (int32_t*)(uintptr_t)result,
                                              (uint32_t*)(uintptr_t)(g->own + kPeerStatusOffset), kPeerTimeoutNs, reset, reset_value, stream);
    if (krc != 0) return set_err(3, krc, "basalt_k_peer_allreduce_max_i32", basalt_k_last_error());
    return 0;
}

int basalt_rt_peer_max_i32(basalt_rt_peer_group* g, uint64_t shard, int64_t n, uint64_t result, void* stream) {
    if (!g || !shard || !result) return set_err(4, 0, "basalt_rt_peer_max_i32", "null argument");
    if (!g->connected) return set_err(4, 0, "basalt_rt_peer_max_i32", "the group is not connected");
    int rc = make_current(g->ctx);
    if (rc) return rc;
    if (++g->epoch == 0) g->epoch = 1;
    int krc = basalt_k_max_i32_allreduce((const int32_t*)(uintptr_t)shard, n, (int32_t*)(uintptr_t)(g->own + kPeerPartialOffset), g->inbox, g->nranks, g->rank, g->epoch,
                                         (int32_t*)(uintptr_t)result, (uint32_t*)(uintptr_t)(g->own + kPeerStatusOffset),
                                         (uint32_t*)(uintptr_t)(g->own + kPeerTicketOffset), kPeerTimeoutNs, stream);
    if (krc != 0) return set_err(3, krc, "basalt_k_max_i32_allreduce", basalt_k_last_error());
    return 0;
}

int basalt_rt_peer_group_status(basalt_rt_peer_group* g, uint32_t* status_out) {
    if (!g || !status_out) return set_err(4, 0, "basalt_rt_peer_group_status", "null argument");
    int rc = make_current(g->ctx);
    if (rc) return rc;
    const Fns& f = g->ctx->drv->f;
    rc = check(f, "cuCtxSynchronize", f.cuCtxSynchronize());
    if (rc) return rc;
    return check(f, "cuMemcpyDtoH", f.cuMemcpyDtoH(status_out, g->own + kPeerStatusOffset, 4));
}

int basalt_rt_peer_group_destroy(basalt_rt_peer_group* g) {
    if (!g) return 0;
    int rc = make_current(g->ctx);
    const Fns& f = g->ctx->drv->f;
    if (!rc) {
        f.cuCtxSynchronize();
        for (int r = 0; r < g->nranks; r++)
            if (r != g->rank && g->inbox[r]) f.cuIpcCloseMemHandle((CUdeviceptr)g->inbox[r]);
        f.cuMemFree(g->own);
    }
    delete g;
    return rc;
}

}  // extern "C"
