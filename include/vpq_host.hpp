// vpq_host.hpp -- C++ host layer over the C ABI (vpq.h) with the names and call shapes of the
// reference's metal-compute classes, so a model family's dispatch code (and its tests) port by
// substitution. Header-only; needs the CUDA runtime for buffers and streams.
//
//   reference (apple-silicon/metal-compute)                 here (namespace vpq::host)
//   MetalCompute::load_library(name)      metal-compute.h:301   Compute::load_library
//   ComputeLibrary::function(entry)       compute-library.h:134 ComputeLibrary::function
//   MetalCompute::make_shared_buffer(n)   shared-buffer.h:33    Compute::make_shared_buffer
//   CommandStream::begin_compute()        command-stream.h      CommandStream::begin_compute
//   ComputeEncoder::set_function / set_buffer / set_constant / dispatch
//                                         compute-encoder.h:80-83,188
//   CommandStream::commit().wait()        command-stream.h:144  CommandStream::commit().wait()
//   Fence::wait_ok(&reason)               command-stream.h:92-99 Fence::wait_ok
//   AffineQuantizer::quantize_linear      generative-models/quantize/affine-quantizer.cc:52-84
//
// Differences kept visible: SharedBuffer is CUDA managed memory (contents() is host-visible like
// Apple's unified memory; production code would use device buffers), and dispatch() takes no grid:
// the launch geometry is derived from K / N / M.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>
#include <utility>

#include "vpq.h"

namespace vpq {
namespace host {

// Move-only buffer visible to host and device (the reference's SharedBuffer, shared-buffer.h:33-175).
class SharedBuffer {
 public:
  SharedBuffer() = default;
  explicit SharedBuffer(std::size_t bytes) : _bytes(bytes) {
    if (bytes == 0 || cudaMallocManaged(&_ptr, bytes) != cudaSuccess) {
      cudaGetLastError();
      _ptr = nullptr;
      _bytes = 0;
    }
  }
  SharedBuffer(SharedBuffer&& o) noexcept : _ptr(o._ptr), _bytes(o._bytes) { o._ptr = nullptr; o._bytes = 0; }
  SharedBuffer& operator=(SharedBuffer&& o) noexcept {
    if (this != &o) {
      reset();
      _ptr = o._ptr;
      _bytes = o._bytes;
      o._ptr = nullptr;
      o._bytes = 0;
    }
    return *this;
  }
  SharedBuffer(const SharedBuffer&) = delete;
  SharedBuffer& operator=(const SharedBuffer&) = delete;
  ~SharedBuffer() { reset(); }

  bool empty() const noexcept { return _ptr == nullptr; }
  void* contents() const noexcept { return _ptr; }
  std::size_t size() const noexcept { return _bytes; }

 private:
  void reset() {
    if (_ptr) { cudaFree(_ptr); }
    _ptr = nullptr;
    _bytes = 0;
  }
  void* _ptr = nullptr;
  std::size_t _bytes = 0;
};

// A kernel entry of a library; invalid if the (library, entry) pair is unknown.
class ComputeFunction {
 public:
  ComputeFunction() = default;
  explicit ComputeFunction(const vpq_function* fn) : _fn(fn) {}
  bool valid() const noexcept { return _fn != nullptr; }
  const vpq_function* handle() const noexcept { return _fn; }

 private:
  const vpq_function* _fn = nullptr;
};

class ComputeLibrary {
 public:
  ComputeLibrary() = default;
  explicit ComputeLibrary(std::string name) : _name(std::move(name)) {}
  ComputeFunction function(const char* entry) const {
    return ComputeFunction(vpq_function_lookup(_name.c_str(), entry));
  }
  const std::string& name() const noexcept { return _name; }

 private:
  std::string _name;
};

// Completion handle of a committed stream.
class Fence {
 public:
  Fence(cudaStream_t st, int enqueue_status) : _st(st), _status(enqueue_status) {}
  void wait() { wait_ok(nullptr); }
  // false if an enqueue failed, the stream faulted, or a bounded device-side wait gave up
  bool wait_ok(std::string* reason) {
    if (_status != VPQ_OK) {
      if (reason) { *reason = vpq_last_error(); }
      return false;
    }
    const cudaError_t e = cudaStreamSynchronize(_st);
    if (e != cudaSuccess) {
      if (reason) { *reason = cudaGetErrorString(e); }
      return false;
    }
    uint32_t detail = 0;
    if (vpq_device_status(_st, &detail) != VPQ_OK) {
      if (reason) { *reason = vpq_last_error(); }
      return false;
    }
    return true;
  }

 private:
  cudaStream_t _st;
  int _status;
};

class CommandStream;

// Binds slots and dispatches one kernel at a time into the stream (single-threaded, like the
// reference's encoder). An unbound slot is reported as an error, not a silent wrong answer.
class ComputeEncoder {
 public:
  void set_function(const ComputeFunction& fn) { _fn = fn; }
  void set_buffer(int index, const SharedBuffer& buf, std::size_t byte_offset = 0) {
    if (index >= 0 && index < 12) { _args.buffers[index] = static_cast<const char*>(buf.contents()) + byte_offset; }
  }
  void set_buffer(int index, const void* device_ptr) {
    if (index >= 0 && index < 12) { _args.buffers[index] = device_ptr; }
  }
  // The reference numbers the int constants after the buffers: QMV 5:K 6:N (7: residual buffer of
  // _add, total rows of _batch), QMM 5:K 6:N 7:M, dequant 4:K 5:N, quant 4:K 5:N 6:clip.
  // set_k / set_n / set_m / set_clip say which is which.
  void set_k(int64_t K) { _args.K = K; }
  void set_n(int64_t N) { _args.N = N; }
  void set_m(int64_t M) { _args.M = M; }
  void set_clip(float clip) { _args.clip = clip; }
  // affine_qmv_qkv_w4g64 numbers its constants 7:K 8:q_rows 9:k_rows 10:v_rows (outputs in slots 4..6)
  // affine_qmm_swiglu_w4g64_bm64_rs: constants 8:out_stride 9:out_off
  void set_out_block(int64_t out_stride, int64_t out_off) {
    _args.out_stride = out_stride;
    _args.out_off = out_off;
  }
  // the grouped GEMMs: experts in w; rows of y (down) or of the hidden (gate|up)
  void set_grouped(int64_t experts, int64_t rows) {
    _args.experts = experts;
    _args.rows = rows;
  }
  // the gathered expert GEMVs: experts in w, pairs per token (gate|up); the norm + q|k|v GEMV: epsilon
  void set_gather(int64_t experts, int64_t top_k) {
    _args.experts = experts;
    _args.top_k = top_k;
  }
  void set_eps(float eps) { _args.eps = eps; }
  void set_qkv_rows(int64_t q_rows, int64_t k_rows, int64_t v_rows) {
    _args.q_rows = q_rows;
    _args.k_rows = k_rows;
    _args.v_rows = v_rows;
  }
  void dispatch();

 private:
  friend class CommandStream;
  explicit ComputeEncoder(CommandStream* s) : _stream(s) { _args = vpq_dispatch_args(); _args.M = 1; _args.clip = 1.0f; }
  CommandStream* _stream;
  ComputeFunction _fn;
  vpq_dispatch_args _args;
};

class CommandStream {
 public:
  CommandStream() {
    if (cudaStreamCreateWithFlags(&_st, cudaStreamNonBlocking) != cudaSuccess) {
      cudaGetLastError();
      _st = nullptr;
      _valid = false;
    }
  }
  ~CommandStream() {
    if (_st) { cudaStreamDestroy(_st); }
  }
  CommandStream(const CommandStream&) = delete;
  CommandStream& operator=(const CommandStream&) = delete;
  bool valid() const noexcept { return _valid; }
  ComputeEncoder begin_compute() { return ComputeEncoder(this); }
  Fence commit() {
    const int s = _status;
    _status = VPQ_OK;
    return Fence(_st, s);
  }
  cudaStream_t native() const noexcept { return _st; }

 private:
  friend class ComputeEncoder;
  cudaStream_t _st = nullptr;
  bool _valid = true;
  int _status = VPQ_OK;  // first enqueue error since the last commit
};

inline void ComputeEncoder::dispatch() {
  int rc = _fn.valid() ? vpq_dispatch(_fn.handle(), &_args, _stream->_st) : VPQ_ERR_NOT_FOUND;
  if (rc != VPQ_OK && _stream->_status == VPQ_OK) { _stream->_status = rc; }
}

// The device object (the reference's MetalCompute, metal-compute.h:32-36).
class Compute {
 public:
  bool valid() const {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
      cudaGetLastError();
      return false;
    }
    return true;
  }
  ComputeLibrary load_library(const char* name) const { return ComputeLibrary(name); }
  SharedBuffer make_shared_buffer(std::size_t bytes) const { return SharedBuffer(bytes); }
};

// generative-models/quantize/affine-quantizer.h:20-52, for bits = 4, group = 64.
class AffineQuantizer {
 public:
  explicit AffineQuantizer(Compute* mc) : _mc(mc), _ok(mc != nullptr && mc->valid()) {
    if (_ok) {
      _fn[0] = mc->load_library("affine_dequant").function("affine_quant_w4_g64");
      _fn[1] = mc->load_library("affine_dequant_bf16").function("affine_quant_w4_g64");
      _ok = _fn[0].valid() && _fn[1].valid();
    }
  }
  bool valid() const noexcept { return _ok; }
  static std::size_t weight_bytes(int N, int K, int bits) { return vpq_weight_bytes(N, K, bits); }
  static std::size_t scale_bytes(int N, int K, int group) { return vpq_scale_bytes(N, K, group); }

  // Quantize w_in[N,K] into freshly allocated (w_out U32, s_out F16, b_out F16); one
  // self-contained stream (commit + wait). Returns false on bad arguments.
  bool quantize_linear(const SharedBuffer& w_in, bool src_bf16, int N, int K, int bits, int group, float clip,
                       SharedBuffer& w_out, SharedBuffer& s_out, SharedBuffer& b_out) const {
    if (!_ok || N <= 0 || K <= 0 || bits != 4 || group != 64 || (K % group) != 0) { return false; }
    w_out = _mc->make_shared_buffer(weight_bytes(N, K, bits));
    s_out = _mc->make_shared_buffer(scale_bytes(N, K, group));
    b_out = _mc->make_shared_buffer(scale_bytes(N, K, group));
    if (w_out.empty() || s_out.empty() || b_out.empty()) { return false; }
    CommandStream stream;
    if (!stream.valid()) { return false; }
    {
      ComputeEncoder enc = stream.begin_compute();
      enc.set_function(_fn[src_bf16 ? 1 : 0]);
      enc.set_buffer(0, w_in);
      enc.set_buffer(1, w_out);
      enc.set_buffer(2, s_out);
      enc.set_buffer(3, b_out);
      enc.set_k(K);
      enc.set_n(N);
      enc.set_clip(clip);
      enc.dispatch();
    }
    return stream.commit().wait_ok(nullptr);
  }

 private:
  Compute* _mc;
  ComputeFunction _fn[2];
  bool _ok;
};

}  // namespace host
}  // namespace vpq
