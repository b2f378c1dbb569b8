// sb_frontend_device_noalloc: the batched log-mel frontend for callers that must not allocate.
//
// The ordinary entry points (sb_frontend_device, sb_transcribe_chunks, ...) keep grow-only work
// buffers inside an sb_ctx and enlarge them with cudaMalloc / cudaFree when a batch is bigger than
// any before.  Two kinds of caller cannot live with that:
//   * an ingest thread that extracts features while another stream of the same GPU is busy
//     encoding or decoding: cudaMalloc and cudaFree synchronise the whole device, so one growing
//     buffer stalls every stream at an unpredictable moment;
//   * a host program that has handed all device memory to its own pool (an inference server, a
//     framework allocator) and gives a library nothing but the input and output buffers it names.
// For them this file holds everything the frontend needs besides its input and output in ONE
// file-scope device array of fixed size: the constant tables (Hann window, mel taps, twiddles) and the
// per-clip metadata (start, length, first output row) that the kernel reads; the per-feature statistics
// stay inside the kernel's CTAs.  Every GPU that loads the library carries this array (about 32 KB)
// until the process exits.
//
// Consequences the caller has to know:
//   * at most kNoAllocMaxClips clips per call; more is refused with SB_INVALID_ARGUMENT;
//   * the first call on a device resolves the array's device address and fills the tables; make
//     that first call outside any stream capture.  First calls from several host threads are
//     serialised by a mutex.  A call made while its stream is capturing is refused with
//     SB_INVALID_ARGUMENT: the per-call clip metadata is copied from the host stack;
//   * all calls on a device share the array, and it keeps what the last call left in it.  Nothing in
//     it has to start at zero (each call rewrites the metadata of the clips it processes before its
//     kernel reads them), but two calls whose kernels overlap on the GPU, from different streams or
//     threads, race on it: serialise them;
//   * no cudaMalloc, cudaFree or allocating library routine is called, on the first call or later.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <climits>
#include <cstring>
#include <mutex>
#include <string>

#include "context.h"
#include "frontend.h"

namespace sb {

constexpr int kNoAllocMaxClips = 1024;

namespace {

// Layout of the scratch array (all offsets multiples of 256 bytes).
constexpr size_t kTablesBytes = (sizeof(FrontendTables) + 255) / 256 * 256;
constexpr size_t kMetaBytes = (3 * (size_t)(kNoAllocMaxClips + 1) * sizeof(int64_t) + 255) / 256 * 256;
constexpr size_t kScratchBytes = kTablesBytes + kMetaBytes;

static __device__ __align__(256) unsigned char g_frontend_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
// Device address of g_frontend_scratch per device.  The symbol's name is only a host-side handle:
// kernels must be given the address that cudaGetSymbolAddress returns for the current device.
unsigned char* g_scratch_ptr[kMaxDevices] = {};
std::atomic<bool> g_ready[kMaxDevices];
std::mutex g_setup_mutex;  // first calls from several host threads (same or different devices) take turns

int32_t setup_device(int device, cudaStream_t stream) {
    if (g_ready[device].load(std::memory_order_acquire)) return SB_OK;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_ready[device].load(std::memory_order_acquire)) return SB_OK;
    unsigned char* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_frontend_scratch);
    if (e != cudaSuccess || !ptr) return cuda_fail(e != cudaSuccess ? e : cudaErrorInvalidSymbol, "cudaGetSymbolAddress(frontend scratch)");
    e = frontend_configure();  // shared-memory opt-in of the log-mel kernel; not an allocation
    if (e != cudaSuccess) return cuda_fail(e, "frontend_configure");
    static FrontendTables host_tables;  // static: the copy below may outlive this call; guarded by the mutex
    if (!build_frontend_tables(&host_tables, nullptr))
        return fail(SB_INVALID_MODEL_OUTPUT, "mel filterbank rows exceed the tap budget");
    e = cudaMemcpyAsync(ptr, &host_tables, sizeof(FrontendTables), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return cuda_fail(e, "copy of the frontend tables");
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return cuda_fail(e, "frontend table set-up");
    g_scratch_ptr[device] = ptr;
    g_ready[device].store(true, std::memory_order_release);  // published after the address it guards
    return SB_OK;
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" int32_t sb_frontend_device_noalloc(const float* d_pcm, const int64_t* clip_offsets, int64_t n_clips,
                                              float preemphasis, int32_t normalize, float* d_feats,
                                              int64_t* frame_offsets, void* stream) {
    if (!d_pcm || !clip_offsets || !d_feats) return fail(SB_INVALID_ARGUMENT, "null argument");
    if (n_clips <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");
    if (n_clips > kNoAllocMaxClips)
        return fail(SB_INVALID_ARGUMENT, "sb_frontend_device_noalloc takes at most " + std::to_string(kNoAllocMaxClips) +
                                             " clips per call (its scratch memory has a fixed size); got " +
                                             std::to_string(n_clips));
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (device < 0 || device >= kMaxDevices) return fail(SB_INVALID_ARGUMENT, "device index out of range");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The clip metadata below is copied from this call's stack frame; a capturing stream would record that host
    // address and read it again at every replay, long after the frame is gone.  Refuse instead.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing(st, &cap);
    if (e != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
        if (e != cudaSuccess) (void)cudaGetLastError();
        return fail(SB_INVALID_ARGUMENT, "sb_frontend_device_noalloc was called while a stream capture is active; "
                                         "it copies per-call metadata from the host stack and refuses to be recorded");
    }
    int32_t s = setup_device(device, st);
    if (s != SB_OK) return s;

    // metadata on the stack: starts | lengths | output-row prefix sums
    const size_t n1 = (size_t)kNoAllocMaxClips + 1;
    int64_t meta[3 * (kNoAllocMaxClips + 1)] = {};
    int64_t* fo = meta + 2 * n1;
    fo[0] = 0;
    for (int64_t i = 0; i < n_clips; ++i) {
        const int64_t len = clip_offsets[i + 1] - clip_offsets[i];
        if (len <= 0) return fail(SB_EMPTY_AUDIO, "audio input was empty");
        meta[i] = clip_offsets[i];
        meta[n1 + i] = len;
        const int64_t t = frames_for_samples(len);
        if (t > INT32_MAX / 2) return fail(SB_INVALID_ARGUMENT, "clip too long");
        fo[i + 1] = fo[i] + t;
    }
    if (frame_offsets) std::memcpy(frame_offsets, fo, sizeof(int64_t) * ((size_t)n_clips + 1));

    unsigned char* base = g_scratch_ptr[device];
    const FrontendTables* d_tables = reinterpret_cast<const FrontendTables*>(base);
    int64_t* d_meta = reinterpret_cast<int64_t*>(base + kTablesBytes);
    // pageable source: the runtime has staged the bytes by the time the call returns
    e = cudaMemcpyAsync(d_meta, meta, sizeof(meta), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_fail(e, "copy of the clip metadata");
    e = frontend_launch(d_pcm, kSampleF32, d_meta, d_meta + n1, d_meta + 2 * n1, (int)n_clips, preemphasis, d_tables,
                        d_feats, normalize != 0, st);
    if (e == cudaErrorMisalignedAddress) return fail(SB_INVALID_ARGUMENT, "the feature buffer must be 16-byte aligned");
    if (e != cudaSuccess) return cuda_fail(e, "frontend launch");
    return SB_OK;
}
