// Engine object: device binding, status word, launch counter, tensor-map encoder.
// Plays the part that VoxCPMBackend's CUDA initialisation (src/backend.cpp:146-205) and
// ggml-cuda's per-context state play for the reference's attention path.
#include "common.cuh"

#include <cstdlib>
#include <cstring>
#include <new>

namespace vox {

static thread_local char g_error[512] = "";

void set_error(const char * fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

// Developer settings come from the environment exactly once per process (the first engine created reads them);
// nothing on a launch path calls getenv.
static int env_int(const char * name) {
    const char * s = getenv(name);
    return s ? atoi(s) : 0;
}
static bool g_pdl_on = true;

bool pdl_enabled() { return g_pdl_on; }

void reset_ticket_counters(vox_engine * e, cudaStream_t stream);

int make_tensor_map(const vox_engine * e, CUtensorMap * out, void * base, CUtensorMapDataType dt, const uint64_t dims[5],
                    const uint64_t strides[4], const uint32_t box[5], CUtensorMapSwizzle swizzle) {
    VOX_REQUIRE(e && e->encode, VOX_ATTN_CUDA_ERROR, "tensor-map encoder unavailable");
    VOX_REQUIRE((reinterpret_cast<uintptr_t>(base) & 15) == 0, VOX_ATTN_INVALID_ARGUMENT,
                "base address must be 16-byte aligned for bulk-tensor copies");
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], estr[5] = {1, 1, 1, 1, 1};
    for (int i = 0; i < 5; ++i) { d[i] = dims[i]; b[i] = box[i]; }
    for (int i = 0; i < 4; ++i) {
        VOX_REQUIRE(strides[i] % 16 == 0, VOX_ATTN_INVALID_ARGUMENT,
                    "stride %d (%llu bytes) must be a multiple of 16 bytes for bulk-tensor copies", i + 1,
                    (unsigned long long) strides[i]);
        s[i] = strides[i];
    }
    CUresult rc = e->encode(out, dt, 5, base, d, s, b, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    VOX_REQUIRE(rc == CUDA_SUCCESS, VOX_ATTN_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code %d", (int) rc);
    return VOX_ATTN_OK;
}

}  // namespace vox

using namespace vox;

namespace {

// The path every kernel takes when a copy or a peer never shows up, exercised on purpose: one thread waits,
// with the given limit, on a barrier that nothing arrives at, gives up, raises the status word and returns.
__global__ void wait_that_runs_out_kernel(int * status, long long limit_cycles) {
    __shared__ uint64_t bar;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        fence_mbar_init();
        if (!mbar_wait_bounded(b, 0, limit_cycles)) atomicOr(status, kStatusTimeout);
    }
}

}  // namespace

extern "C" {

const char * vox_attn_last_error_string(void) { return g_error; }

const char * vox_attn_status_string(int status) {
    switch (status) {
        case VOX_ATTN_OK: return "ok";
        case VOX_ATTN_INVALID_ARGUMENT: return "invalid argument";
        case VOX_ATTN_UNSUPPORTED: return "unsupported";
        case VOX_ATTN_WORKSPACE_TOO_SMALL: return "workspace too small";
        case VOX_ATTN_CUDA_ERROR: return "CUDA error";
        case VOX_ATTN_TIMEOUT: return "device-side wait timed out";
        case VOX_ATTN_OUT_OF_MEMORY: return "out of memory";
        case VOX_ATTN_DEVICE_STATE: return "device-side state does not fit the call";
        default: return "unknown status";
    }
}

int vox_engine_create(int device, vox_engine ** out) {
    VOX_REQUIRE(out != nullptr, VOX_ATTN_INVALID_ARGUMENT, "vox_engine_create: out is null");
    *out = nullptr;
    int n_dev = 0;
    VOX_CUDA_TRY(cudaGetDeviceCount(&n_dev));
    VOX_REQUIRE(device >= 0 && device < n_dev, VOX_ATTN_INVALID_ARGUMENT, "device %d out of range (%d devices)", device,
                n_dev);
    cudaDeviceProp prop;
    VOX_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    VOX_REQUIRE(prop.major == 10, VOX_ATTN_UNSUPPORTED,
                "device %d is compute capability %d.%d; this engine is built for sm_100a only", device, prop.major,
                prop.minor);
    VOX_CUDA_TRY(cudaSetDevice(device));

    vox_engine * e = new (std::nothrow) vox_engine();
    VOX_REQUIRE(e != nullptr, VOX_ATTN_OUT_OF_MEMORY, "out of host memory");
    e->device   = device;
    e->sm_count = prop.multiProcessorCount;
    {
        const char * s = getenv("VOX_NO_PDL");
        g_pdl_on = !(s && s[0] == '1');
        e->decode_wave[0] = env_int("VOX_DECODE_WAVE");
        e->decode_wave[1] = env_int("VOX_DECODE_WAVE_Q8");
        e->linear_split   = env_int("VOX_LINEAR_SPLIT");
        if (getenv("VOX_DECODE_CLUSTER") != nullptr) e->decode_cluster = env_int("VOX_DECODE_CLUSTER");
        if (getenv("VOX_DECODE_EARLY") != nullptr) e->decode_early_tiles = env_int("VOX_DECODE_EARLY");
        const char * w = getenv("VOX_PREFILL_WEIGHTS");
        e->prefill_single_f16 = (w && w[0] == 'f') ? 1 : 0;
    }

    cudaError_t err = cudaHostAlloc(reinterpret_cast<void **>(&e->status_host), sizeof(int) * 4, cudaHostAllocMapped);
    if (err == cudaSuccess) {
        memset(e->status_host, 0, sizeof(int) * 4);
        err = cudaHostGetDevicePointer(reinterpret_cast<void **>(&e->status_dev), e->status_host, 0);
    }
    if (err != cudaSuccess) {
        set_error("status word allocation failed: %s", cudaGetErrorString(err));
        delete e;
        return VOX_ATTN_CUDA_ERROR;
    }

    void *                          fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (err != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
        set_error("cuTensorMapEncodeTiled not available from the driver");
        cudaFreeHost(e->status_host);
        delete e;
        return VOX_ATTN_CUDA_ERROR;
    }
    e->encode = reinterpret_cast<encode_tiled_fn>(fn);
    err = cudaMalloc(reinterpret_cast<void **>(&e->counters_dev), sizeof(int) * kCounterSlots);
    if (err == cudaSuccess) err = cudaMemset(e->counters_dev, 0, sizeof(int) * kCounterSlots);
    if (err != cudaSuccess) {
        set_error("ticket counter allocation failed: %s", cudaGetErrorString(err));
        cudaGetLastError();
        if (e->counters_dev) cudaFree(e->counters_dev);
        cudaFreeHost(e->status_host);
        delete e;
        return VOX_ATTN_OUT_OF_MEMORY;
    }
    *out      = e;
    return VOX_ATTN_OK;
}

void vox_engine_destroy(vox_engine * e) {
    if (!e) return;
    cudaSetDevice(e->device);
    if (e->stage_dev) cudaFree(e->stage_dev);
    if (e->stage_ws) cudaFree(e->stage_ws);
    if (e->counters_dev) cudaFree(e->counters_dev);
    if (e->status_host) cudaFreeHost(e->status_host);
    delete e;
}

uint64_t vox_engine_launch_count(const vox_engine * e) { return e ? e->launches : 0; }

int vox_engine_selftest_wait(vox_engine * e, long long limit_cycles, void * stream) {
    VOX_REQUIRE(e != nullptr, VOX_ATTN_INVALID_ARGUMENT, "engine is null");
    VOX_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000000LL, VOX_ATTN_INVALID_ARGUMENT,
                "limit_cycles must be in (0, 2e9] (about a second at most)");
    VOX_CUDA_TRY(cudaSetDevice(e->device));
    wait_that_runs_out_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(e->status_dev, limit_cycles);
    return check_launch(e, "wait_that_runs_out_kernel");
}

int vox_engine_sync_status(vox_engine * e, void * stream) {
    VOX_REQUIRE(e != nullptr, VOX_ATTN_INVALID_ARGUMENT, "engine is null");
    VOX_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    const int word = *reinterpret_cast<volatile int *>(e->status_host);
    if (word != 0) {
        *reinterpret_cast<volatile int *>(e->status_host) = 0;
        reset_ticket_counters(e, static_cast<cudaStream_t>(stream));  // a kernel that gave up may have left tickets behind
        if (word & kStatusTimeout) {
            set_error("device status word 0x%x: a bounded wait on a copy barrier ran out", word);
            return VOX_ATTN_TIMEOUT;
        }
        set_error("device status word 0x%x: a kernel found a stream longer than its cache rows; that row was not stored", word);
        return VOX_ATTN_DEVICE_STATE;
    }
    return VOX_ATTN_OK;
}

}  // extern "C"
