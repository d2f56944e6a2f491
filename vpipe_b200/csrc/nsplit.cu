// nsplit.cu -- column-split QMM over the GPUs of one box.
//
// The reference is single-GPU, so this part has no counterpart there. Output
// columns are independent: rank r owns rows [r*N/G, (r+1)*N/G) of the packed
// weight, scales and biases (contiguous slices of all three arrays, the same
// property the reference uses to row-concatenate q|k|v,
// generative-models/qwen3/metal-qwen-model.cc:214-250), x is replicated, and
// the only exchange is an all-gather of the output column blocks over
// NVLink / NVSwitch. NCCL is loaded with dlopen so the library itself has no
// link-time dependency on it.
//
// Each rank's GEMM writes its [M, N/G] block contiguously into a shard-major
// buffer [G, M, N/G]. With m_chunks > 1 the rows are cut into chunks and the
// exchange of chunk i (grouped ncclSend / ncclRecv, which may place every
// peer's rows anywhere) runs on a second stream while chunk i+1 is computed.
#include "vpq_common.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

struct vpq_sym_buf {
  void* local = nullptr;
  void* peer[8] = {};   // peer[r]: rank r's buffer mapped here (peer[rank] == local)
  size_t bytes = 0;
};

struct vpq_comm_s {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1, device = 0;
  // fused column-split: symmetric buffers, and a flag array per rank for the cross-GPU barrier
  vpq_sym_buf bufs[8];
  int nbufs = 0;
  vpq_sym_buf flags;       // uint32 per rank: [r] rank r started call `epoch`, [8 + r] rank r finished it; [16] sender-CTA
                           // count; [32 ..) one counter per GEMM tile
  uint32_t epoch = 0;
  void* handle_stage = nullptr;  // device staging for the IPC-handle exchange
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ev_start = nullptr, ev_done = nullptr;
  cudaEvent_t ev_chunk[16] = {};
};

namespace vpq {
namespace {

constexpr int kTileFlags = 1 << 18;  // GEMM tiles the fused column split can count (1 MB of flags per GPU)
constexpr int kCollectiveSms = 16;  // SMs the GEMM leaves to NCCL when the exchange overlaps it

struct Nccl {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

Nccl& nccl() {
  static Nccl n;
  static bool tried = false;
  if (!tried) {
    tried = true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* nm : names) {
      n.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
      if (n.handle) { break; }
    }
    if (n.handle) {
#define VPQ_SYM(field, sym) n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.handle, sym))
      VPQ_SYM(GetUniqueId, "ncclGetUniqueId");
      VPQ_SYM(CommInitRank, "ncclCommInitRank");
      VPQ_SYM(CommDestroy, "ncclCommDestroy");
      VPQ_SYM(AllGather, "ncclAllGather");
      VPQ_SYM(Send, "ncclSend");
      VPQ_SYM(Recv, "ncclRecv");
      VPQ_SYM(GroupStart, "ncclGroupStart");
      VPQ_SYM(GroupEnd, "ncclGroupEnd");
      VPQ_SYM(GetErrorString, "ncclGetErrorString");
#undef VPQ_SYM
      n.ok = n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.AllGather && n.Send && n.Recv &&
             n.GroupStart && n.GroupEnd && n.GetErrorString;
    }
  }
  return n;
}

#define VPQ_NCCL_OK(expr)                                                              \
  do {                                                                                 \
    ncclResult_t _r = (expr);                                                          \
    if (_r != ncclSuccess) {                                                           \
      return ::vpq::fail(VPQ_ERR_NCCL, "%s: %s", #expr, nccl().GetErrorString(_r));    \
    }                                                                                  \
  } while (0)

// Cross-GPU barrier over peer-mapped flags: thread r publishes this rank's epoch into rank r's
// flag array, then waits (bounded) until rank r's epoch has arrived here. Launched after the
// GEMM on the same stream, so this GPU's peer stores are complete before its flag is raised.
// `max_polls` bounds the wait (about 100 ns per poll); a rank that never arrives is recorded in
// the status word and the kernel returns.
constexpr uint32_t kBarrierPolls = 1u << 24;
__global__ void peer_barrier_kernel(uint32_t* const* peer_flags, uint32_t* my_flags, int rank, int world,
                                    uint32_t epoch, uint32_t* status, uint32_t max_polls) {
  const int r = threadIdx.x;
  if (r >= world) { return; }
  __threadfence_system();
  volatile uint32_t* remote = peer_flags[r] + rank;
  *remote = epoch;
  __threadfence_system();
  volatile uint32_t* mine = my_flags + r;
  for (uint32_t i = 0; i < max_polls; ++i) {
    if ((int32_t)(*mine - epoch) >= 0) { return; }
    __nanosleep(100);
  }
  atomicCAS(status, 0u, 0x7700u | (uint32_t)r);  // rank r never arrived
}

// The waiting half alone: thread r waits (bounded) until flags[r] has reached `epoch`.
__global__ void peer_wait_kernel(uint32_t* flags, int rank, int world, uint32_t epoch, uint32_t* status,
                                 uint32_t max_polls) {
  const int r = threadIdx.x;
  if (r >= world || r == rank) { return; }
  volatile uint32_t* f = flags + r;
  for (uint32_t i = 0; i < max_polls; ++i) {
    if ((int32_t)(*f - epoch) >= 0) {
      __threadfence_system();
      return;
    }
    __nanosleep(100);
  }
  atomicCAS(status, 0u, 0x7700u | (uint32_t)r);  // rank r never finished
}

__device__ uint32_t g_nsplit_status;

// shard-major [G, M, Ns] -> row-major [M, G*Ns] for rows [m0, m1)
__global__ void __launch_bounds__(256)
shards_to_rowmajor_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int64_t M,
                          int ns_vec, int world, int64_t m0, int64_t m1) {
  const int64_t per_row = (int64_t)ns_vec * world;
  const int64_t total = (m1 - m0) * per_row;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t m = m0 + i / per_row;
    const int64_t c = i % per_row;
    const int r = (int)(c / ns_vec);
    const int j = (int)(c % ns_vec);
    out[m * per_row + c] = in[((int64_t)r * M + m) * ns_vec + j];
  }
}

}  // namespace
}  // namespace vpq

using namespace vpq;

namespace {
void unmap_peers(vpq_comm* c, vpq_sym_buf* b);
}

extern "C" int vpq_comm_unique_id(void* id_host) {
  clear_error();
  if (!id_host) { return fail(VPQ_ERR_INVALID_ARG, "comm_unique_id: null pointer"); }
  if (!nccl().ok) { return fail(VPQ_ERR_NCCL, "libnccl.so.2 could not be loaded"); }
  static_assert(sizeof(ncclUniqueId) == VPQ_UNIQUE_ID_BYTES, "unique id size");
  ncclUniqueId id;
  VPQ_NCCL_OK(nccl().GetUniqueId(&id));
  std::memcpy(id_host, &id, sizeof(id));
  return VPQ_OK;
}

extern "C" int vpq_comm_create(const void* id_host, int rank, int world, vpq_comm** out) {
  clear_error();
  if (!id_host || !out || world < 1 || rank < 0 || rank >= world) {
    return fail(VPQ_ERR_INVALID_ARG, "comm_create: bad arguments (rank=%d world=%d)", rank, world);
  }
  if (!nccl().ok) { return fail(VPQ_ERR_NCCL, "libnccl.so.2 could not be loaded"); }
  if (int rc = require_sm100()) { return rc; }
  vpq_comm* c = new vpq_comm_s();
  c->rank = rank;
  c->world = world;
  VPQ_CUDA_OK(cudaGetDevice(&c->device));
  ncclUniqueId id;
  std::memcpy(&id, id_host, sizeof(id));
  ncclResult_t r = nccl().CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) {
    delete c;
    return fail(VPQ_ERR_NCCL, "ncclCommInitRank: %s", nccl().GetErrorString(r));
  }
  VPQ_CUDA_OK(cudaStreamCreateWithFlags(&c->comm_stream, cudaStreamNonBlocking));
  VPQ_CUDA_OK(cudaEventCreateWithFlags(&c->ev_start, cudaEventDisableTiming));
  VPQ_CUDA_OK(cudaEventCreateWithFlags(&c->ev_done, cudaEventDisableTiming));
  for (auto& e : c->ev_chunk) { VPQ_CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming)); }
  *out = c;
  return VPQ_OK;
}

extern "C" int vpq_comm_destroy(vpq_comm* c) {
  clear_error();
  if (!c) { return VPQ_OK; }
  if (c->comm_stream) { cudaStreamSynchronize(c->comm_stream); }
  cudaDeviceSynchronize();
  for (int i = 0; i < c->nbufs; ++i) { unmap_peers(c, &c->bufs[i]); }
  if (c->flags.local) { unmap_peers(c, &c->flags); }
  if (c->handle_stage) { cudaFree(c->handle_stage); }
  if (c->comm) { nccl().CommDestroy(c->comm); }
  for (auto& e : c->ev_chunk) {
    if (e) { cudaEventDestroy(e); }
  }
  if (c->ev_start) { cudaEventDestroy(c->ev_start); }
  if (c->ev_done) { cudaEventDestroy(c->ev_done); }
  if (c->comm_stream) { cudaStreamDestroy(c->comm_stream); }
  delete c;
  return VPQ_OK;
}

extern "C" int vpq_comm_rank(const vpq_comm* c) { return c ? c->rank : -1; }
extern "C" int vpq_comm_world(const vpq_comm* c) { return c ? c->world : 0; }

extern "C" int vpq_affine_qmm_w4g64_bf16_nsplit(vpq_comm* c, const uint32_t* w_shard,
                                                const void* scales_shard, const void* biases_shard,
                                                const void* x, void* y_shards, void* y_rowmajor,
                                                int64_t K, int64_t N, int64_t M, int m_chunks,
                                                void* stream) {
  clear_error();
  if (!c || !y_shards) { return fail(VPQ_ERR_INVALID_ARG, "qmm_nsplit: null communicator or output"); }
  const int G = c->world;
  if (N <= 0 || (N % G) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "qmm_nsplit: N=%lld is not a multiple of the %d ranks",
                (long long)N, G);
  }
  if (m_chunks < 1 || m_chunks > 16) {
    return fail(VPQ_ERR_INVALID_ARG, "qmm_nsplit: m_chunks must be 1..16 (got %d)", m_chunks);
  }
  const int64_t Ns = N / G;
  if (y_rowmajor && (Ns % 8) != 0) {
    return fail(VPQ_ERR_UNSUPPORTED, "qmm_nsplit: row-major output needs N/world %% 8 == 0");
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  __nv_bfloat16* ys = static_cast<__nv_bfloat16*>(y_shards);
  __nv_bfloat16* mine = ys + (int64_t)c->rank * M * Ns;

  if (G == 1) {
    if (int rc = vpq_affine_qmm_w4g64_bf16(w_shard, scales_shard, biases_shard, x, mine, K, Ns, M, stream)) {
      return rc;
    }
    if (y_rowmajor && y_rowmajor != y_shards) {
      VPQ_CUDA_OK(cudaMemcpyAsync(y_rowmajor, y_shards, (size_t)M * N * 2, cudaMemcpyDeviceToDevice, st));
    }
    return VPQ_OK;
  }

  // chunk boundaries on multiples of 256 rows (the GEMM's row tile)
  const int64_t row_tiles = (M + 255) / 256;
  if (m_chunks > row_tiles) { m_chunks = (int)row_tiles; }
  const uint16_t* xb = static_cast<const uint16_t*>(x);
  for (int ch = 0; ch < m_chunks; ++ch) {
    const int64_t m0 = (row_tiles * ch / m_chunks) * 256;
    int64_t m1 = (row_tiles * (ch + 1) / m_chunks) * 256;
    if (m1 > M) { m1 = M; }
    const int64_t rows = m1 - m0;
    if (rows <= 0) { continue; }
    // chunked: leave a few SMs idle so the exchange of the previous chunk runs beside this GEMM
    const int reserve = m_chunks > 1 ? kCollectiveSms : 0;
    if (int rc = qmm_launch_reserved(w_shard, scales_shard, biases_shard, xb + m0 * K, mine + m0 * Ns, K, Ns,
                                     rows, stream, reserve)) {
      return rc;
    }
    VPQ_CUDA_OK(cudaEventRecord(c->ev_chunk[ch], st));
    VPQ_CUDA_OK(cudaStreamWaitEvent(c->comm_stream, c->ev_chunk[ch], 0));
    if (m_chunks == 1) {
      VPQ_NCCL_OK(nccl().AllGather(mine, ys, (size_t)(M * Ns), ncclBfloat16, c->comm, c->comm_stream));
    } else {
      VPQ_NCCL_OK(nccl().GroupStart());
      for (int r = 0; r < G; ++r) {
        if (r == c->rank) { continue; }
        VPQ_NCCL_OK(nccl().Send(mine + m0 * Ns, (size_t)(rows * Ns), ncclBfloat16, r, c->comm, c->comm_stream));
        VPQ_NCCL_OK(nccl().Recv(ys + ((int64_t)r * M + m0) * Ns, (size_t)(rows * Ns), ncclBfloat16, r,
                                c->comm, c->comm_stream));
      }
      VPQ_NCCL_OK(nccl().GroupEnd());
    }
    if (y_rowmajor) {
      const int64_t vecs = rows * (N / 8);
      int64_t blocks = (vecs + 255) / 256;
      const int64_t cap = (int64_t)num_sms() * 8;
      if (blocks > cap) { blocks = cap; }
      shards_to_rowmajor_kernel<<<(unsigned)blocks, 256, 0, c->comm_stream>>>(
          reinterpret_cast<const uint4*>(ys), reinterpret_cast<uint4*>(y_rowmajor), M, (int)(Ns / 8), G,
          m0, m1);
      VPQ_LAUNCH_OK("shards_to_rowmajor");
    }
  }
  VPQ_CUDA_OK(cudaEventRecord(c->ev_done, c->comm_stream));
  VPQ_CUDA_OK(cudaStreamWaitEvent(st, c->ev_done, 0));
  return VPQ_OK;
}

// ------------------------------------------------------------ fused column-split
namespace {

// Collective: every rank maps every other rank's `local` allocation (CUDA IPC; one process per GPU).
int map_peers(vpq_comm* c, vpq_sym_buf* b) {
  const int G = c->world;
  cudaIpcMemHandle_t mine;
  VPQ_CUDA_OK(cudaIpcGetMemHandle(&mine, b->local));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!c->handle_stage) { VPQ_CUDA_OK(cudaMalloc(&c->handle_stage, 64 * 10)); }  // 8 + 1 handles, pointer table
  char* stage = static_cast<char*>(c->handle_stage);
  VPQ_CUDA_OK(cudaMemcpyAsync(stage + 64 * 8, &mine, 64, cudaMemcpyHostToDevice, c->comm_stream));
  VPQ_NCCL_OK(nccl().AllGather(stage + 64 * 8, stage, 64, ncclUint8, c->comm, c->comm_stream));
  cudaIpcMemHandle_t all[8];
  VPQ_CUDA_OK(cudaMemcpyAsync(all, stage, 64 * (size_t)G, cudaMemcpyDeviceToHost, c->comm_stream));
  VPQ_CUDA_OK(cudaStreamSynchronize(c->comm_stream));
  for (int r = 0; r < G; ++r) {
    if (r == c->rank) {
      b->peer[r] = b->local;
    } else {
      VPQ_CUDA_OK(cudaIpcOpenMemHandle(&b->peer[r], all[r], cudaIpcMemLazyEnablePeerAccess));
    }
  }
  return VPQ_OK;
}

void unmap_peers(vpq_comm* c, vpq_sym_buf* b) {
  for (int r = 0; r < c->world; ++r) {
    if (r != c->rank && b->peer[r]) { cudaIpcCloseMemHandle(b->peer[r]); }
    b->peer[r] = nullptr;
  }
  if (b->local) { cudaFree(b->local); }
  b->local = nullptr;
}

}  // namespace

extern "C" int vpq_comm_alloc_symmetric(vpq_comm* c, size_t bytes, void** local_ptr) {
  clear_error();
  if (!c || !local_ptr || bytes == 0) { return fail(VPQ_ERR_INVALID_ARG, "comm_alloc_symmetric: bad arguments"); }
  if (c->world > 8) { return fail(VPQ_ERR_UNSUPPORTED, "comm_alloc_symmetric: at most 8 ranks"); }
  if (c->nbufs >= 8) { return fail(VPQ_ERR_UNSUPPORTED, "comm_alloc_symmetric: at most 8 live buffers"); }
  if (!c->flags.local) {  // first use: the barrier flags
    VPQ_CUDA_OK(cudaMalloc(&c->flags.local, (32 + kTileFlags) * sizeof(uint32_t)));
    VPQ_CUDA_OK(cudaMemset(c->flags.local, 0, (32 + kTileFlags) * sizeof(uint32_t)));
    VPQ_CUDA_OK(cudaDeviceSynchronize());
    c->flags.bytes = (32 + kTileFlags) * sizeof(uint32_t);
    if (int rc = map_peers(c, &c->flags)) { return rc; }
    // the peers' flag arrays as a device table for the barrier kernel
    uint32_t* hp[8] = {};
    for (int r = 0; r < c->world; ++r) { hp[r] = static_cast<uint32_t*>(c->flags.peer[r]); }
    VPQ_CUDA_OK(cudaMemcpy(static_cast<char*>(c->handle_stage) + 64 * 9, hp, sizeof(hp), cudaMemcpyHostToDevice));
  }
  vpq_sym_buf* b = &c->bufs[c->nbufs];
  VPQ_CUDA_OK(cudaMalloc(&b->local, bytes));
  b->bytes = bytes;
  if (int rc = map_peers(c, b)) { return rc; }
  ++c->nbufs;
  *local_ptr = b->local;
  return VPQ_OK;
}

extern "C" int vpq_comm_free_symmetric(vpq_comm* c, void* local_ptr) {
  clear_error();
  if (!c || !local_ptr) { return fail(VPQ_ERR_INVALID_ARG, "comm_free_symmetric: bad arguments"); }
  for (int i = 0; i < c->nbufs; ++i) {
    if (c->bufs[i].local == local_ptr) {
      cudaDeviceSynchronize();
      unmap_peers(c, &c->bufs[i]);
      c->bufs[i] = c->bufs[c->nbufs - 1];
      c->bufs[c->nbufs - 1] = vpq_sym_buf();
      --c->nbufs;
      return VPQ_OK;
    }
  }
  return fail(VPQ_ERR_INVALID_ARG, "comm_free_symmetric: not a buffer of this communicator");
}

extern "C" int vpq_affine_qmm_w4g64_bf16_nsplit_fused(vpq_comm* c, const uint32_t* w_shard,
                                                      const void* scales_shard, const void* biases_shard,
                                                      const void* x, void* y_sym, int64_t K, int64_t N,
                                                      int64_t M, void* stream) {
  clear_error();
  if (!c || !y_sym) { return fail(VPQ_ERR_INVALID_ARG, "qmm_nsplit_fused: null communicator or output"); }
  const int G = c->world;
  if (N <= 0 || (N % (8 * G)) != 0) {
    return fail(VPQ_ERR_INVALID_ARG, "qmm_nsplit_fused: N=%lld must be a multiple of 8 x %d ranks", (long long)N, G);
  }
  const vpq_sym_buf* b = nullptr;
  for (int i = 0; i < c->nbufs; ++i) {
    if (c->bufs[i].local == y_sym) { b = &c->bufs[i]; }
  }
  if (!b) { return fail(VPQ_ERR_INVALID_ARG, "qmm_nsplit_fused: y must come from vpq_comm_alloc_symmetric"); }
  if (b->bytes < (size_t)M * (size_t)N * 2) { return fail(VPQ_ERR_INVALID_ARG, "qmm_nsplit_fused: y too small"); }
  const int64_t Ns = N / G;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // this GPU's copy first, then the peers' (rotated, so that the ranks do not all start on the same peer)
  void* dests[8];
  PeerSync ps = {};
  int n = 0;
  dests[n++] = b->local;
  for (int r = 1; r < G; ++r) {
    const int peer = (c->rank + r) % G;
    ps.flag_of[n] = static_cast<uint32_t*>(c->flags.peer[peer]);
    ps.src_rank[n] = peer;
    dests[n++] = b->peer[peer];
  }
  ps.my_flags = static_cast<uint32_t*>(c->flags.local);
  ps.warps_done = ps.my_flags + 16;
  ps.tile_flags = ps.my_flags + 32;
  ps.tile_flag_count = kTileFlags;
  ps.epoch = ++c->epoch;
  ps.rank = c->rank;
  // The handshake with the peers runs inside the GEMM kernel: it announces "started" when it starts,
  // its sender warps hold their stores into a peer's y until that peer has started too (whatever the
  // peer enqueued earlier to read y is then done), and the sender warp that finishes last announces
  // "finished" to every peer.
  if (int rc = qmm_launch_multi_dest(w_shard, scales_shard, biases_shard, x, dests, n, N, (int64_t)c->rank * Ns,
                                     K, Ns, M, stream, G > 1 ? &ps : nullptr)) {
    return rc;
  }
  if (G > 1) {
    // y is complete on this GPU once every peer has announced "finished": a small kernel behind the
    // GEMM waits for that (bounded), so that later work on the stream sees all column blocks.
    uint32_t* status = nullptr;
    VPQ_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_nsplit_status));
    peer_wait_kernel<<<1, 32, 0, st>>>(ps.my_flags + 8, c->rank, G, ps.epoch, status, kBarrierPolls);
    VPQ_LAUNCH_OK("peer_wait");
  }
  return VPQ_OK;
}

// The cross-GPU flag barrier run on ONE GPU against a rank that never arrives: `workspace` (256
// bytes of device memory) plays every rank's flag table, rank 0 publishes its epoch, and the wait for
// `absent_rank` runs out after max_polls polls (about 100 ns each). Nothing faults or hangs: the
// kernel records 0x7700 | absent_rank and returns; vpq_device_status then reports VPQ_ERR_TIMEOUT
// with detail 0x20000 | 0x7700 | absent_rank and clears the word.
extern "C" int vpq_peer_barrier_probe(void* workspace, int world, int absent_rank, uint32_t max_polls, void* stream) {
  clear_error();
  if (!workspace || world < 2 || world > 8 || absent_rank < 1 || absent_rank >= world) {
    return fail(VPQ_ERR_INVALID_ARG, "peer_barrier_probe: need a workspace, 2 <= world <= 8, 1 <= absent_rank < world");
  }
  if (max_polls == 0 || max_polls > (1u << 20)) {
    return fail(VPQ_ERR_INVALID_ARG, "peer_barrier_probe: 0 < max_polls <= 2^20 (the probe must end in a fraction of a second)");
  }
  if (reinterpret_cast<uintptr_t>(workspace) & 15) { return fail(VPQ_ERR_ALIGNMENT, "peer_barrier_probe: workspace alignment"); }
  if (int rc = require_sm100()) { return rc; }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* ws = static_cast<char*>(workspace);
  uint32_t* flags = reinterpret_cast<uint32_t*>(ws + 64);
  // every rank's table is this one; the entries of the ranks that "arrived" carry the epoch already
  uint32_t host_flags[8] = {};
  for (int r = 0; r < world; ++r) { host_flags[r] = (r == absent_rank) ? 0u : 1u; }
  uint32_t* host_ptrs[8];
  for (int r = 0; r < 8; ++r) { host_ptrs[r] = flags; }
  VPQ_CUDA_OK(cudaMemcpyAsync(ws, host_ptrs, sizeof(host_ptrs), cudaMemcpyHostToDevice, st));
  VPQ_CUDA_OK(cudaMemcpyAsync(flags, host_flags, sizeof(host_flags), cudaMemcpyHostToDevice, st));
  VPQ_CUDA_OK(cudaStreamSynchronize(st));  // the copies read this call's stack
  uint32_t* status = nullptr;
  VPQ_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_nsplit_status));
  peer_barrier_kernel<<<1, 32, 0, st>>>(reinterpret_cast<uint32_t* const*>(ws), flags, 0, world, 1u, status, max_polls);
  VPQ_LAUNCH_OK("peer_barrier (probe)");
  return VPQ_OK;
}

namespace vpq {
int nsplit_status_read(cudaStream_t st, uint32_t* out) {
  uint32_t v = 0;
  VPQ_CUDA_OK(cudaMemcpyFromSymbolAsync(&v, g_nsplit_status, sizeof(v), 0, cudaMemcpyDeviceToHost, st));
  VPQ_CUDA_OK(cudaStreamSynchronize(st));
  if (v != 0) {
    const uint32_t zero = 0;
    VPQ_CUDA_OK(cudaMemcpyToSymbolAsync(g_nsplit_status, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, st));
    VPQ_CUDA_OK(cudaStreamSynchronize(st));
  }
  *out = v;
  return VPQ_OK;
}
}  // namespace vpq
