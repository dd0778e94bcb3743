// One-directional peer channel between two pipeline-adjacent GPUs.
//
// Replaces the reference's per-tensor helper threads and their
// GPU -> CPU -> TCP -> CPU -> GPU path (runtime/communication.py:610-712) with a
// ring of slots that lives in the CONSUMER's HBM and is mapped into the producer
// process with CUDA IPC.  A push is three stream-ordered operations on the
// producer's side stream: wait for a free slot, copy the payload over NVLink
// (copy engine), publish a sequence number.  A receive mirrors it on the
// consumer.  Shapes travel in a 64-byte header in the same slot (the reference
// sends a separate int32 shape message first, communication.py:664-669).
//
//   base + 0    : uint64 produced   (written by the producer, polled locally by the consumer)
//   base + 64   : uint64 consumed   (written by the consumer, polled over NVLink by the producer)
//   base + 256 + i * slot_stride : slot i = 64-byte header + payload
//
// Every device-side wait is bounded; when the bound runs out the kernel records
// PD_ERR_TIMEOUT in the channel's status word and returns, so the context stays
// usable and the host learns of a dead peer instead of hanging.  Once the status
// word is set the channel is dead: later waits return at once, payloads are no
// longer copied into slots the consumer has not freed, nothing more is published
// or released, and a receive fills its destination with zeros.  The same happens
// when a message's byte count differs from what the receiver asked for
// (PD_ERR_INVALID).  The status is mirrored into pinned host memory, so the host
// can look at it between launches without synchronising anything.
#include "pd_common.cuh"
#include <cstring>
#include <new>

namespace {

constexpr int kHeaderBytes = 64;
constexpr int kControlBytes = 256;
constexpr int kMaxDims = 5;

struct PdChan {
  int producer;            // 1 = this end pushes, 0 = this end receives
  int owner;               // 1 = this end allocated the ring
  int ipc_mapped;          // 1 = base came from cudaIpcOpenMemHandle
  int device;
  uint8_t* base;
  int64_t slot_bytes;      // payload capacity
  int64_t slot_stride;
  int num_slots;
  unsigned long long seq;  // sequence number of the next push / receive (1-based)
  int* status;             // device word: 0 ok, PD_ERR_TIMEOUT after a wait ran out, PD_ERR_INVALID on a size mismatch
  int* host_flag;          // pinned host mirror of *status (host pointer)
  int* host_flag_dev;      // the same word as the device sees it
  long long timeout_cycles;
};

struct ExportBlob {          // what pd_chan_export_handle writes (128 bytes)
  cudaIpcMemHandle_t mem;    // 64 bytes
  int64_t slot_bytes;
  int64_t slot_stride;
  int32_t num_slots;
  int32_t device;
  char pad[128 - 64 - 8 - 8 - 4 - 4];
};
static_assert(sizeof(ExportBlob) == 128, "export blob is 128 bytes");

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void chan_fail(int* status, int* host_flag, int code) {
  if (atomicCAS(status, 0, code) == 0) {
    *(volatile int*)host_flag = code;
    __threadfence_system();
  }
}

// Spins until *counter >= need or the cycle budget runs out.  A channel that has already failed is not waited on.
__global__ void chan_wait_kernel(const unsigned long long* counter, unsigned long long need,
                                 long long timeout_cycles, int* status, int* host_flag) {
  if (*(volatile int*)status != 0) return;
  const long long t0 = clock64();
  while (ld_acquire_sys(counter) < need) {
    if (clock64() - t0 > timeout_cycles) {
      chan_fail(status, host_flag, PD_ERR_TIMEOUT);
      return;
    }
    __nanosleep(200);
  }
}

struct Header { long long v[8]; };   // seq, nbytes, ndim, dims[5]

// Payload copy that does nothing on a failed channel.  mode 0 (push): plain copy.  mode 1 (receive): `header`
// is the slot header; a byte count other than `bytes` fails the channel, and on a failed channel dst is
// zero-filled so that what the stage computes next is at least deterministic.
__global__ void chan_copy_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, long long bytes,
                                 int mode, const Header* header, int* status, int* host_flag) {
  bool dead = *(volatile int*)status != 0;
  if (!dead && mode == 1 && header->v[1] != bytes) {
    if (blockIdx.x == 0 && threadIdx.x == 0) chan_fail(status, host_flag, PD_ERR_INVALID);
    dead = true;
  }
  if (dead && mode == 0) return;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const bool vec = ((((uintptr_t)dst) | ((uintptr_t)src)) & 15) == 0;
  const long long nvec = vec ? bytes / 16 : 0;
  if (dead) {
    for (long long i = tid; i < nvec; i += nthreads) reinterpret_cast<uint4*>(dst)[i] = make_uint4(0, 0, 0, 0);
    for (long long i = nvec * 16 + tid; i < bytes; i += nthreads) dst[i] = 0;
    return;
  }
  for (long long i = tid; i < nvec; i += nthreads) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  for (long long i = nvec * 16 + tid; i < bytes; i += nthreads) dst[i] = src[i];
}

__global__ void chan_publish_kernel(Header* slot_header, Header h, unsigned long long* produced,
                                    unsigned long long seq, const int* status) {
  if (*(volatile const int*)status != 0) return;            // nothing is published on a failed channel
  *slot_header = h;
  __threadfence_system();
  st_release_sys(produced, seq);
}

__global__ void chan_release_kernel(unsigned long long* consumed, unsigned long long seq, const int* status) {
  if (*(volatile const int*)status != 0) return;            // a failed receive does not free the slot
  __threadfence_system();
  st_release_sys(consumed, seq);
}

void chan_free(PdChan* c) {
  if (!c) return;
  if (c->status) cudaFree(c->status);
  if (c->host_flag) cudaFreeHost(c->host_flag);
  if (c->ipc_mapped && c->base) cudaIpcCloseMemHandle(c->base);
  else if (c->owner && c->base) cudaFree(c->base);
  delete c;
}

int chan_alloc_status(PdChan* c) {
  PD_CUDA(cudaMalloc((void**)&c->status, 256));
  PD_CUDA(cudaMemset(c->status, 0, 256));
  PD_CUDA(cudaHostAlloc((void**)&c->host_flag, 64, cudaHostAllocMapped));
  *c->host_flag = 0;
  PD_CUDA(cudaHostGetDevicePointer((void**)&c->host_flag_dev, c->host_flag, 0));
  return PD_OK;
}

int copy_grid(long long bytes) {
  long long blocks = (bytes / 16 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 64) blocks = 64;       // enough to fill NVLink / HBM, few enough to leave the SMs to the stage
  return (int)blocks;
}

long long cycles_for_ms(int device, int timeout_ms) {
  int khz = 0;
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device) != cudaSuccess || khz <= 0) khz = 1900000;
  return (long long)khz * (long long)timeout_ms;
}

}  // namespace

// Consumer side: allocates the ring (set-up time; nothing on the data path allocates).
PD_EXPORT int pd_chan_create(int64_t slot_bytes, int num_slots, int timeout_ms, void** chan) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(chan && slot_bytes > 0 && num_slots >= 1 && num_slots <= 64 && timeout_ms > 0, "pd_chan_create: bad arguments");
  PdChan* c = new (std::nothrow) PdChan();
  PD_REQUIRE(c, "pd_chan_create: out of host memory");
  memset(c, 0, sizeof(*c));
  PD_CUDA(cudaGetDevice(&c->device));
  c->producer = 0; c->owner = 1;
  c->slot_bytes = slot_bytes;
  c->slot_stride = kHeaderBytes + ((slot_bytes + 255) / 256) * 256;
  c->num_slots = num_slots;
  c->seq = 1;
  c->timeout_cycles = cycles_for_ms(c->device, timeout_ms);
  const size_t total = kControlBytes + (size_t)c->slot_stride * num_slots;
  cudaError_t e = cudaMalloc((void**)&c->base, total);
  if (e == cudaSuccess) e = cudaMemset(c->base, 0, kControlBytes);
  if (e != cudaSuccess) {
    pd_set_error("pd_chan_create: allocating %zu bytes failed: %s", total, cudaGetErrorString(e));
    chan_free(c);
    return PD_ERR_CUDA;
  }
  rc = chan_alloc_status(c);
  if (rc == PD_OK && cudaDeviceSynchronize() != cudaSuccess) { pd_set_error("pd_chan_create: synchronise failed"); rc = PD_ERR_CUDA; }
  if (rc != PD_OK) { chan_free(c); return rc; }
  *chan = c;
  return PD_OK;
}

// 128-byte blob (HOST memory) to hand to the producer process.
PD_EXPORT int pd_chan_export_handle(void* chan, void* blob128) {
  PD_REQUIRE(chan && blob128, "pd_chan_export_handle: null argument");
  PdChan* c = (PdChan*)chan;
  PD_REQUIRE(c->owner && !c->producer, "pd_chan_export_handle: only the consumer end exports");
  ExportBlob b;
  memset(&b, 0, sizeof(b));
  PD_CUDA(cudaIpcGetMemHandle(&b.mem, c->base));
  b.slot_bytes = c->slot_bytes; b.slot_stride = c->slot_stride; b.num_slots = c->num_slots; b.device = c->device;
  memcpy(blob128, &b, sizeof(b));
  return PD_OK;
}

// Producer side, in another process: maps the consumer's ring.
PD_EXPORT int pd_chan_open(const void* blob128, int timeout_ms, void** chan) {
  int rc = pd_check_device();
  if (rc != PD_OK) return rc;
  PD_REQUIRE(blob128 && chan && timeout_ms > 0, "pd_chan_open: bad arguments");
  ExportBlob b;
  memcpy(&b, blob128, sizeof(b));
  PD_REQUIRE(b.slot_bytes > 0 && b.num_slots >= 1 && b.num_slots <= 64, "pd_chan_open: corrupt handle blob");
  PdChan* c = new (std::nothrow) PdChan();
  PD_REQUIRE(c, "pd_chan_open: out of host memory");
  memset(c, 0, sizeof(*c));
  PD_CUDA(cudaGetDevice(&c->device));
  c->producer = 1; c->owner = 0; c->ipc_mapped = 1;
  c->slot_bytes = b.slot_bytes; c->slot_stride = b.slot_stride; c->num_slots = b.num_slots;
  c->seq = 1;
  c->timeout_cycles = cycles_for_ms(c->device, timeout_ms);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, b.mem, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    pd_set_error("cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
    delete c;
    return PD_ERR_CUDA;
  }
  c->base = (uint8_t*)p;
  rc = chan_alloc_status(c);
  if (rc != PD_OK) { chan_free(c); return rc; }
  *chan = c;
  return PD_OK;
}

// Producer end over the same memory inside one process (single-GPU tests of the protocol).
PD_EXPORT int pd_chan_open_local(void* consumer_chan, int timeout_ms, void** chan) {
  PD_REQUIRE(consumer_chan && chan && timeout_ms > 0, "pd_chan_open_local: bad arguments");
  PdChan* src = (PdChan*)consumer_chan;
  PdChan* c = new (std::nothrow) PdChan();
  PD_REQUIRE(c, "pd_chan_open_local: out of host memory");
  *c = *src;
  c->producer = 1; c->owner = 0; c->ipc_mapped = 0; c->seq = 1;
  c->status = nullptr; c->host_flag = nullptr; c->host_flag_dev = nullptr;
  c->timeout_cycles = cycles_for_ms(c->device, timeout_ms);
  int rc = chan_alloc_status(c);
  if (rc != PD_OK) { chan_free(c); return rc; }
  *chan = c;
  return PD_OK;
}

// Enqueue on `stream`: wait for a free slot, copy `bytes` from src, publish.  dims: HOST array.
PD_EXPORT int pd_chan_push(void* chan, const void* src, int64_t bytes, int ndim, const int64_t* dims,
                           void* stream) {
  PD_REQUIRE(chan && src && bytes >= 0 && ndim >= 0 && ndim <= kMaxDims && (ndim == 0 || dims), "pd_chan_push: bad arguments");
  PdChan* c = (PdChan*)chan;
  PD_REQUIRE(c->producer, "pd_chan_push: not a producer end");
  PD_REQUIRE(bytes <= c->slot_bytes, "pd_chan_push: %lld bytes exceed the slot capacity %lld", (long long)bytes, (long long)c->slot_bytes);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned long long* produced = (unsigned long long*)(c->base);
  unsigned long long* consumed = (unsigned long long*)(c->base + 64);
  const unsigned long long seq = c->seq;
  uint8_t* slot = c->base + kControlBytes + (int64_t)((seq - 1) % c->num_slots) * c->slot_stride;
  if (seq > (unsigned long long)c->num_slots) {
    chan_wait_kernel<<<1, 1, 0, s>>>(consumed, seq - c->num_slots, c->timeout_cycles, c->status, c->host_flag_dev);
    PD_LAUNCH_CHECK("chan_wait_kernel");
  }
  if (bytes > 0) {
    chan_copy_kernel<<<copy_grid(bytes), 256, 0, s>>>(slot + kHeaderBytes, (const uint8_t*)src, bytes, 0, nullptr, c->status,
                                                     c->host_flag_dev);
    PD_LAUNCH_CHECK("chan_copy_kernel");
  }
  Header h;
  memset(&h, 0, sizeof(h));
  h.v[0] = (long long)seq; h.v[1] = bytes; h.v[2] = ndim;
  for (int i = 0; i < ndim; ++i) h.v[3 + i] = dims[i];
  chan_publish_kernel<<<1, 1, 0, s>>>((Header*)slot, h, produced, seq, c->status);
  PD_LAUNCH_CHECK("chan_publish_kernel");
  c->seq = seq + 1;
  return PD_OK;
}

// Enqueue on `stream`: wait for the next message, copy `bytes` of its payload to dst, free the slot.
PD_EXPORT int pd_chan_wait(void* chan, void* dst, int64_t bytes, void* stream) {
  PD_REQUIRE(chan && (dst || bytes == 0) && bytes >= 0, "pd_chan_wait: bad arguments");
  PdChan* c = (PdChan*)chan;
  PD_REQUIRE(!c->producer, "pd_chan_wait: not a consumer end");
  PD_REQUIRE(bytes <= c->slot_bytes, "pd_chan_wait: %lld bytes exceed the slot capacity %lld", (long long)bytes, (long long)c->slot_bytes);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned long long* produced = (unsigned long long*)(c->base);
  unsigned long long* consumed = (unsigned long long*)(c->base + 64);
  const unsigned long long seq = c->seq;
  uint8_t* slot = c->base + kControlBytes + (int64_t)((seq - 1) % c->num_slots) * c->slot_stride;
  chan_wait_kernel<<<1, 1, 0, s>>>(produced, seq, c->timeout_cycles, c->status, c->host_flag_dev);
  PD_LAUNCH_CHECK("chan_wait_kernel");
  chan_copy_kernel<<<copy_grid(bytes), 256, 0, s>>>((uint8_t*)dst, slot + kHeaderBytes, bytes, 1, (const Header*)slot, c->status,
                                                   c->host_flag_dev);
  PD_LAUNCH_CHECK("chan_copy_kernel");
  chan_release_kernel<<<1, 1, 0, s>>>(consumed, seq, c->status);
  PD_LAUNCH_CHECK("chan_release_kernel");
  c->seq = seq + 1;
  return PD_OK;
}

// Blocks the host until the next message has arrived (or the bound ran out) and returns its header:
// out8 (HOST) = {seq, nbytes, ndim, d0..d4}.  For tensors whose shape changes per minibatch.
PD_EXPORT int pd_chan_peek_header(void* chan, int64_t* out8, void* stream) {
  PD_REQUIRE(chan && out8, "pd_chan_peek_header: null argument");
  PdChan* c = (PdChan*)chan;
  PD_REQUIRE(!c->producer, "pd_chan_peek_header: not a consumer end");
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned long long seq = c->seq;
  uint8_t* slot = c->base + kControlBytes + (int64_t)((seq - 1) % c->num_slots) * c->slot_stride;
  chan_wait_kernel<<<1, 1, 0, s>>>((unsigned long long*)c->base, seq, c->timeout_cycles, c->status, c->host_flag_dev);
  PD_LAUNCH_CHECK("chan_wait_kernel");
  PD_CUDA(cudaMemcpyAsync(out8, slot, 64, cudaMemcpyDeviceToHost, s));
  int st = 0;
  PD_CUDA(cudaMemcpyAsync(&st, c->status, sizeof(int), cudaMemcpyDeviceToHost, s));
  PD_CUDA(cudaStreamSynchronize(s));
  if (st != 0) {
    pd_set_error("pd_chan_peek_header: no message within the wait bound (peer stalled or gone)");
    return PD_ERR_TIMEOUT;
  }
  return PD_OK;
}

namespace {
int report_status(int st) {
  if (st == PD_ERR_INVALID) {
    pd_set_error("peer channel: a message's byte count differs from what the receiver asked for "
                 "(tensor shape or dtype tables of the two stages disagree)");
    return PD_ERR_INVALID;
  }
  pd_set_error("peer channel: a bounded device wait ran out (peer stalled or gone)");
  return PD_ERR_TIMEOUT;
}
}  // namespace

// Synchronises `stream` and reports the channel status: 0, PD_ERR_TIMEOUT or PD_ERR_INVALID.  A failed channel
// stays failed (its sequence numbers no longer match its peer's); close it and open a new one.
PD_EXPORT int pd_chan_status(void* chan, void* stream) {
  PD_REQUIRE(chan, "pd_chan_status: null channel");
  PdChan* c = (PdChan*)chan;
  cudaStream_t s = (cudaStream_t)stream;
  int st = 0;
  PD_CUDA(cudaMemcpyAsync(&st, c->status, sizeof(int), cudaMemcpyDeviceToHost, s));
  PD_CUDA(cudaStreamSynchronize(s));
  return st != 0 ? report_status(st) : PD_OK;
}

// The same status without touching any stream: reads the pinned host mirror the kernels write on failure.
PD_EXPORT int pd_chan_poll(void* chan) {
  PD_REQUIRE(chan, "pd_chan_poll: null channel");
  PdChan* c = (PdChan*)chan;
  const int st = *(volatile int*)c->host_flag;
  return st != 0 ? report_status(st) : PD_OK;
}

PD_EXPORT int pd_chan_close(void* chan) {
  chan_free((PdChan*)chan);
  return PD_OK;
}
