// Owners of the CUDA objects the host engine holds: device and pinned blocks, the activation arena, streams,
// events and instantiated graphs. Each owner frees its object in one place (`drop`), which the destructor and the
// move assignment share; every runtime call is checked through `cuda_check`, which names the call that failed.
#include "qwen38/api.h"

namespace qwen38 {

namespace {

// "<file>:<line>: <call> failed: <runtime's text> (<error name>)"
std::string describe_cuda_failure(cudaError_t code, const char* call, const char* file, int line) {
  std::ostringstream text;
  text << file << ':' << line << ": " << call << " failed: " << cudaGetErrorString(code) << " (" << cudaGetErrorName(code)
       << ')';
  return text.str();
}

void drop_device_block(void*& p) {
  if (p != nullptr) cudaFree(p);
  p = nullptr;
}

void drop_pinned_block(void*& p) {
  if (p != nullptr) cudaFreeHost(p);
  p = nullptr;
}

void drop_graph(cudaGraphExec_t& g) {
  if (g != nullptr) cudaGraphExecDestroy(g);
  g = nullptr;
}

}  // namespace

void cuda_check(cudaError_t err, const char* expr, const char* file, int line) {
  if (err != cudaSuccess) fail(describe_cuda_failure(err, expr, file, line));
}

// ---- device memory ---------------------------------------------------------------------------------
DeviceBuffer::DeviceBuffer(size_t bytes) : bytes_(bytes) {
  if (bytes_ == 0) return;
  QWEN38_CUDA(cudaMalloc(&ptr_, bytes_));
}

DeviceBuffer::~DeviceBuffer() { drop_device_block(ptr_); }

DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& other) noexcept {
  if (this == &other) return *this;
  drop_device_block(ptr_);
  std::swap(ptr_, other.ptr_);
  bytes_ = std::exchange(other.bytes_, 0);
  return *this;
}

void* DeviceArena::allocate(size_t bytes, size_t align) {
  QWEN38_CHECK(align != 0 && (align & (align - 1)) == 0, "arena alignment must be a power of two, got ", align);
  const size_t begin = (used_ + align - 1) & ~(align - 1);
  const size_t end = begin + bytes;
  QWEN38_CHECK(end >= begin && end <= capacity(), "activation arena too small: a request of ", bytes, " bytes at offset ",
               begin, " does not fit into ", capacity(), " bytes");
  used_ = end;
  return block_.as<uint8_t>() + begin;
}

// ---- pinned host memory ------------------------------------------------------------------------------
PinnedBuffer::PinnedBuffer(size_t bytes, bool mapped) : bytes_(bytes), mapped_(mapped) {
  if (bytes_ == 0) return;
  const unsigned flags = mapped_ ? cudaHostAllocMapped : cudaHostAllocDefault;
  QWEN38_CUDA(cudaHostAlloc(&ptr_, bytes_, flags));
}

PinnedBuffer::~PinnedBuffer() { drop_pinned_block(ptr_); }

PinnedBuffer& PinnedBuffer::operator=(PinnedBuffer&& other) noexcept {
  if (this == &other) return *this;
  drop_pinned_block(ptr_);
  std::swap(ptr_, other.ptr_);
  bytes_ = std::exchange(other.bytes_, 0);
  mapped_ = other.mapped_;
  return *this;
}

void* PinnedBuffer::device_ptr() const {
  QWEN38_CHECK(ptr_ != nullptr && mapped_, "only a mapped pinned block has an address on the device");
  void* on_device = nullptr;
  QWEN38_CUDA(cudaHostGetDevicePointer(&on_device, ptr_, 0));
  return on_device;
}

// ---- stream, event -----------------------------------------------------------------------------------
Stream::Stream() { QWEN38_CUDA(cudaStreamCreateWithFlags(&s_, cudaStreamNonBlocking)); }

Stream::~Stream() {
  if (s_ != nullptr) cudaStreamDestroy(s_);
}

void Stream::sync() const { QWEN38_CUDA(cudaStreamSynchronize(s_)); }

Event::Event(bool timing) {
  QWEN38_CUDA(cudaEventCreateWithFlags(&e_, timing ? unsigned(cudaEventDefault) : unsigned(cudaEventDisableTiming)));
}

Event::~Event() {
  if (e_ != nullptr) cudaEventDestroy(e_);
}

void Event::record(cudaStream_t s) const { QWEN38_CUDA(cudaEventRecord(e_, s)); }

void Event::sync() const { QWEN38_CUDA(cudaEventSynchronize(e_)); }

float Event::ms_since(const Event& start) const {
  float elapsed = 0.0f;
  QWEN38_CUDA(cudaEventElapsedTime(&elapsed, start.get(), e_));
  return elapsed;
}

// ---- captured graphs -----------------------------------------------------------------------------------
Graph::~Graph() { drop_graph(exec_); }

Graph& Graph::operator=(Graph&& other) noexcept {
  if (this == &other) return *this;
  drop_graph(exec_);
  std::swap(exec_, other.exec_);
  return *this;
}

// Thread-local capture mode: other host threads (a second engine replica, a loader) may keep calling the runtime.
void Graph::begin_capture(cudaStream_t s) { QWEN38_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal)); }

void Graph::end_capture(cudaStream_t s) {
  cudaGraph_t captured = nullptr;
  QWEN38_CUDA(cudaStreamEndCapture(s, &captured));
  drop_graph(exec_);
  const cudaError_t status = cudaGraphInstantiate(&exec_, captured, 0);
  cudaGraphDestroy(captured);  // the executable graph keeps what it needs
  QWEN38_CUDA(status);
}

void Graph::launch(cudaStream_t s) const {
  QWEN38_CHECK(exec_ != nullptr, "launch of a graph that was never captured");
  QWEN38_CUDA(cudaGraphLaunch(exec_, s));
}

// ---- device properties -----------------------------------------------------------------------------------
DeviceInfo query_device(int device) {
  if (device >= 0) {
    QWEN38_CUDA(cudaSetDevice(device));
  } else {
    QWEN38_CUDA(cudaGetDevice(&device));
  }
  DeviceInfo info;
  info.device = device;
  auto attribute = [device](cudaDeviceAttr which) {
    int value = 0;
    QWEN38_CUDA(cudaDeviceGetAttribute(&value, which, device));
    return value;
  };
  cudaDeviceProp prop{};
  QWEN38_CUDA(cudaGetDeviceProperties(&prop, device));
  info.name = prop.name;
  info.total_mem = prop.totalGlobalMem;
  info.sm_major = attribute(cudaDevAttrComputeCapabilityMajor);
  info.sm_minor = attribute(cudaDevAttrComputeCapabilityMinor);
  info.num_sms = attribute(cudaDevAttrMultiProcessorCount);
  info.l2_bytes = size_t(attribute(cudaDevAttrL2CacheSize));
  info.max_smem_per_block_optin = attribute(cudaDevAttrMaxSharedMemoryPerBlockOptin);
  info.can_map_host = attribute(cudaDevAttrCanMapHostMemory) != 0;
  size_t total_now = 0;
  QWEN38_CUDA(cudaMemGetInfo(&info.free_mem, &total_now));
  return info;
}

}  // namespace qwen38
