// api.cu -- status strings, per-thread error message, device checks, byte-size
// helpers and the (library, entry) function table of the C ABI.
#include "vpq_sm100.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace vpq {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_err[0] = '\0'; }

struct DevInfo {
  int checked = 0;  // 0 = not yet, 1 = ok, -1 = not sm_100
  int major = 0, minor = 0, sms = 0;
};
static DevInfo g_dev[64];
static std::mutex g_dev_mu;

static int probe(int* dev_out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(VPQ_ERR_CUDA, "no usable CUDA device (%s); this library has no CPU path",
                cudaGetErrorString(e));
  }
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DevInfo& d = g_dev[dev];
  if (d.checked == 0) {
    if (cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&d.minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
      cudaGetLastError();
      return fail(VPQ_ERR_CUDA, "cannot query device %d", dev);
    }
    d.checked = (d.major == 10) ? 1 : -1;
  }
  *dev_out = dev;
  return VPQ_OK;
}

int require_sm100() {
  int dev = 0;
  if (int rc = probe(&dev)) { return rc; }
  if (g_dev[dev].checked != 1) {
    return fail(VPQ_ERR_CUDA, "device %d is sm_%d%d; the kernels are built for sm_100a only", dev,
                g_dev[dev].major, g_dev[dev].minor);
  }
  return VPQ_OK;
}

int num_sms() {
  int dev = 0;
  if (probe(&dev) != VPQ_OK) { return 148; }
  return g_dev[dev].sms > 0 ? g_dev[dev].sms : 148;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time, so the library does not link libcuda.
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    } else {
      cudaGetLastError();
    }
  }
  return fn;
}

// Encoding a tensor map costs about a microsecond of host time and a GEMV needs three; a model
// calls the same weights every step, so the maps are kept in a small direct-mapped cache. A map
// is a pure function of the key below, so an entry can never be stale.
namespace {
struct MapKey {
  const void* ptr;
  uint64_t inner, outer, pitch;
  uint32_t box_inner, box_outer;
  int dt, elt_bytes, swz;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && pitch == o.pitch && box_inner == o.box_inner &&
           box_outer == o.box_outer && dt == o.dt && elt_bytes == o.elt_bytes && swz == o.swz;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kMapSlots = 1024;
MapSlot g_maps[kMapSlots];
std::mutex g_maps_mutex;
}  // namespace

int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elt_bytes, const void* ptr,
                uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                CUtensorMapSwizzle swz, const char* what, uint64_t row_pitch_bytes) {
  if (row_pitch_bytes == 0) { row_pitch_bytes = inner * (uint64_t)elt_bytes; }
  const MapKey key = {ptr, inner, outer, row_pitch_bytes, box_inner, box_outer, (int)dt, elt_bytes, (int)swz};
  const uint64_t h = (reinterpret_cast<uintptr_t>(ptr) >> 4) * 0x9E3779B97F4A7C15ull + box_outer * 31u + (uint64_t)dt;
  MapSlot& slot = g_maps[(h >> 32) % kMapSlots];
  {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    if (slot.used && slot.key == key) {
      *map = slot.map;
      return VPQ_OK;
    }
  }
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) { return fail(VPQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver"); }
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(VPQ_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  }
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  slot.key = key;
  slot.map = *map;
  slot.used = true;
  return VPQ_OK;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) only when a launch needs more than any before
// it on this device (the attribute is per function and device; it costs a driver call).
int ensure_dynamic_smem(const void* func, int* granted /* [64], zero-initialised, one per function */, size_t bytes) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { return fail(VPQ_ERR_CUDA, "no current device"); }
  if ((int)bytes <= granted[dev]) { return VPQ_OK; }
  VPQ_CUDA_OK(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  granted[dev] = (int)bytes;
  return VPQ_OK;
}

}  // namespace vpq

using namespace vpq;

extern "C" int vpq_version(void) { return VPQ_VERSION; }

extern "C" const char* vpq_status_string(int status) {
  switch (status) {
    case VPQ_OK: return "ok";
    case VPQ_ERR_INVALID_ARG: return "invalid argument";
    case VPQ_ERR_ALIGNMENT: return "pointer not 16-byte aligned";
    case VPQ_ERR_UNSUPPORTED: return "unsupported shape";
    case VPQ_ERR_CUDA: return "CUDA error or no sm_100 device";
    case VPQ_ERR_NCCL: return "NCCL error";
    case VPQ_ERR_TIMEOUT: return "device-side wait timed out";
    case VPQ_ERR_NOT_FOUND: return "unknown library or entry";
    default: return "unknown status";
  }
}

extern "C" const char* vpq_last_error(void) { return g_err; }

// generative-models/quantize/affine-quantizer.h:37-40
extern "C" size_t vpq_weight_bytes(int N, int K, int bits) {
  return (size_t)N * (size_t)(K * bits / 32) * 4u;
}
extern "C" size_t vpq_scale_bytes(int N, int K, int group) {
  return (size_t)N * (size_t)(K / group) * 2u;
}

// ------------------------------------------------------- function registry
struct vpq_function_s {
  const char* library;
  const char* entry;
  int kind;  // 0 qmv, 1 qmm, 2 dequant, 3 quant(bf16 src), 4 quant(f16 src), 5 qmv+add, 6 qmv swiglu, 7 qmv qkv, 8 qmm swiglu, 9 qmv batch, 58 qmv w8g64, 59 qmm w8g64, 60 qmv w4g32, 61 qmv geglu, 62 qmv gelu*mul, 63 qmm geglu, 64 / 65 qmm swiglu / geglu w8g64, 66..69 qmv w8g64 add / swiglu / qkv / gelu*mul, 70 / 71 qmm swiglu strided store w4 / w8, 72..74 grouped qmm down / swiglu / geglu, 75 qmv norm + qkv, 76..78 gathered expert qmv swiglu / geglu / down, 79..81 qmm w4g32 / geglu w4g32 / w8g32, 82..85 qmv w4g32 add / geglu / gelu*mul / qkv, 86..88 scale-only (Q4_0) qmv w4g32 plain / add / geglu, 89 requant w8 -> w4, 90 qmv geglu w8g64, 91..93 gathered expert qmv w8g64 swiglu / geglu / down, 94 moe gate w8g64, 95 / 96 gathered split-width swiglu (gate w4 + up w8 / gate w8 + up w4), 97..99 grouped qmm w8g64 down / swiglu / geglu, 100 / 101 qmv norm + qkv w8g64 / w4g32, 102 qmv w8g32, 103..106 sorted-slot expert qmv swiglu / down, w4g64 / w8g64, 107 / 108 qmv batch swiglu / geglu; 10 + code: quant / dequant twins (see fmt_*)
};

// The reference selects the element type with the library-name suffix and
// keeps entry names unchanged (apple-silicon/metal-compute/CMakeLists.txt:69-72,156-177).
// The three QMM tile variants share one kernel here (the tile is chosen from
// the shape), so their names all resolve to it.
static const vpq_function_s g_functions[] = {
    {"affine_qmv_bf16", "affine_qmv_w4g64", 0},
    {"affine_qmv_bf16", "affine_qmv_w4g64_r8p2", 0},   // the reference's rows-per-simdgroup tuning twins: same contract
    {"affine_qmv_bf16", "affine_qmv_w8g64_r8p2", 58},
    {"affine_qmv_bf16", "affine_qmv_w4g64_add", 5},
    {"affine_qmv_bf16", "affine_qmv_swiglu_w4g64", 6},
    {"affine_qmv_bf16", "affine_qmv_qkv_w4g64", 7},
    {"affine_qmv_bf16", "affine_qmv_qkv_rms_w4g64", 75},
    {"affine_qmv_bf16", "affine_qmv_qkv_rms_w8g64", 100},
    {"affine_qmv_bf16", "affine_qmv_qkv_rms_w4g32", 101},
    {"affine_qmv_bf16", "affine_gather_qmv_swiglu_w4g64", 76},
    {"affine_qmv_bf16", "affine_gather_qmv_geglu_w4g64", 77},
    {"affine_qmv_bf16", "affine_gather_down_qmv_w4g64", 78},
    {"affine_qmv_bf16", "affine_gather_qmv_swiglu_w8g64", 91},
    {"affine_qmv_bf16", "affine_gather_qmv_geglu_w8g64", 92},
    {"affine_qmv_bf16", "affine_gather_down_qmv_w8g64", 93},
    {"affine_qmv_bf16", "affine_moe_gate_w8g64", 94},
    {"affine_qmv_bf16", "affine_grouped_swiglu_w4g64", 103},
    {"affine_qmv_bf16", "affine_grouped_down_w4g64", 104},
    {"affine_qmv_bf16", "affine_grouped_swiglu_w8g64", 105},
    {"affine_qmv_bf16", "affine_grouped_down_w8g64", 106},
    {"affine_qmv_bf16", "affine_gather_qmv_swiglu_w4w8g64", 95},
    {"affine_qmv_bf16", "affine_gather_qmv_swiglu_w8w4g64", 96},
    {"affine_qmv_bf16", "affine_qmv_geglu_w4g64", 61},
    {"affine_qmv_bf16", "affine_qmv_gelu_mul_w4g64", 62},
    {"affine_qmv_bf16", "affine_qmv_w8g64", 58},
    {"affine_qmv_bf16", "affine_qmv_w8g32", 102},
    {"affine_qmv_bf16", "affine_qmv_w8g64_add", 66},
    {"affine_qmv_bf16", "affine_qmv_swiglu_w8g64", 67},
    {"affine_qmv_bf16", "affine_qmv_qkv_w8g64", 68},
    {"affine_qmv_bf16", "affine_qmv_gelu_mul_w8g64", 69},
    {"affine_qmv_bf16", "affine_qmv_geglu_w8g64", 90},
    {"affine_qmv_bf16", "affine_qmv_w4g32", 60},
    {"affine_qmv_bf16", "affine_qmv_w4g32_add", 82},
    {"affine_qmv_bf16", "affine_qmv_geglu_w4g32", 83},
    {"affine_qmv_bf16", "affine_qmv_gelu_mul_w4g32", 84},
    {"affine_qmv_bf16", "affine_qmv_qkv_w4g32", 85},
    {"affine_qmv_bf16", "affine_qmv_w4g32_q40", 86},
    {"affine_qmv_bf16", "affine_qmv_w4g32_add_q40", 87},
    {"affine_qmv_bf16", "affine_qmv_geglu_w4g32_q40", 88},
    {"affine_qmv_bf16", "affine_qmv_batch_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch4_w4g64", 9},
    // the reference's batch ladder (row-count and tiling twins of one contract: slot 7 = total rows)
    {"affine_qmv_bf16", "affine_qmv_batch4_xp_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch8_tg_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch8_tg4_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch8_xd_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch8_xh_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch8_xh16_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch8_xp1_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch8_xp2_w4g64", 9},
    {"affine_qmv_bf16", "affine_qmv_batch_swiglu_w4g64", 107},
    {"affine_qmv_bf16", "affine_qmv_batch4_swiglu_w4g64", 107},
    {"affine_qmv_bf16", "affine_qmv_batch4_xp_swiglu_w4g64", 107},
    {"affine_qmv_bf16", "affine_qmv_batch8_xp2_swiglu_w4g64", 107},
    {"affine_qmv_bf16", "affine_qmv_batch_geglu_w4g64", 108},
    {"affine_qmv_bf16", "affine_qmv_batch_w8g64", 58},
    {"affine_qmv_bf16", "affine_qmv_batch4_w8g64", 58},
    {"affine_qmv_bf16", "affine_qmv_batch4_xp_w8g64", 58},
    {"affine_qmv_bf16", "affine_qmv_batch8_tg4_w8g64", 58},
    {"affine_qmv_bf16", "affine_qmv_batch8_xd_w8g64", 58},
    {"affine_qmv_bf16", "affine_qmv_batch8_xp2_w8g64", 58},
    {"affine_qmv_bf16", "affine_qmv_batch_w4g32", 60},
    {"affine_qmv_bf16", "affine_qmv_batch_geglu_w4g32", 83},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w4g64", 1},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm64", 1},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm128", 1},
    // the reference's half-precision-accumulate tuning twins: served by the same kernels, which accumulate in f32
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w4g64_bm64_acc16", 1},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w8g64_bm64_acc16", 59},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_acc16", 8},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64_acc16", 8},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_acc16", 64},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm64_acc16", 64},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64_rs_acc16", 70},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm64_rs_acc16", 71},
    {"affine_qmm_mma_bf16", "affine_qmm_mma_w4g64", 1},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w8g64", 59},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w8g64_bm64", 59},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w8g64_bm128", 59},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64", 8},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64", 8},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm128", 8},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w4g64_bm64_rs", 70},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm64_rs", 71},
    {"affine_qmm_steel_bf16", "affine_qmm_grouped_w4g64", 72},
    {"affine_qmm_steel_bf16", "affine_qmm_grouped_swiglu_w4g64", 73},
    {"affine_qmm_steel_bf16", "affine_qmm_grouped_geglu_w4g64", 74},
    {"affine_qmm_steel_bf16", "affine_qmm_grouped_w8g64", 97},
    {"affine_qmm_steel_bf16", "affine_qmm_grouped_swiglu_w8g64", 98},
    {"affine_qmm_steel_bf16", "affine_qmm_grouped_geglu_w8g64", 99},
    {"affine_qmm_steel_bf16", "affine_qmm_geglu_w4g64", 63},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w4g32", 79},
    {"affine_qmm_steel_bf16", "affine_qmm_geglu_w4g32", 80},
    {"affine_qmm_steel_bf16", "affine_qmm_steel_w8g32", 81},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64", 64},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm64", 64},
    {"affine_qmm_steel_bf16", "affine_qmm_swiglu_w8g64_bm128", 64},
    {"affine_qmm_steel_bf16", "affine_qmm_geglu_w8g64", 65},
    {"affine_dequant_bf16", "affine_dequant_w4g64", 2},
    {"affine_dequant_bf16", "affine_quant_w4_g64", 3},
    {"affine_dequant", "affine_quant_w4_g64", 4},
    // the format twins: kind = 10 + 16 * (quant ? 1 + bf16 source : 0) + 4 * (bits == 8) + (group == 32)
    {"affine_dequant_bf16", "affine_dequant_w8g64", 10 + 4},
    {"affine_dequant_bf16", "affine_dequant_w8g32", 10 + 4 + 1},
    {"affine_dequant_bf16", "affine_dequant_w4g32", 10 + 1},
    {"affine_dequant_bf16", "affine_requant_w8_to_w4_g64", 89},
    {"affine_dequant_bf16", "affine_quant_w8_g64", 10 + 32 + 4},
    {"affine_dequant_bf16", "affine_quant_w8_g32", 10 + 32 + 4 + 1},
    {"affine_dequant_bf16", "affine_quant_w4_g32", 10 + 32 + 1},
    {"affine_dequant", "affine_quant_w8_g64", 10 + 16 + 4},
    {"affine_dequant", "affine_quant_w8_g32", 10 + 16 + 4 + 1},
    {"affine_dequant", "affine_quant_w4_g32", 10 + 16 + 1},
};

extern "C" const vpq_function* vpq_function_lookup(const char* library, const char* entry) {
  clear_error();
  if (!library || !entry) {
    fail(VPQ_ERR_NOT_FOUND, "function_lookup: null name");
    return nullptr;
  }
  for (const vpq_function_s& f : g_functions) {
    if (std::strcmp(f.library, library) == 0 && std::strcmp(f.entry, entry) == 0) { return &f; }
  }
  fail(VPQ_ERR_NOT_FOUND, "function_lookup: no entry '%s' in library '%s'", entry, library);
  return nullptr;
}

extern "C" const char* vpq_function_name(const vpq_function* fn) { return fn ? fn->entry : ""; }

extern "C" int vpq_dispatch(const vpq_function* fn, const vpq_dispatch_args* a, void* stream) {
  clear_error();
  if (!fn || !a) { return fail(VPQ_ERR_INVALID_ARG, "dispatch: null function or arguments"); }
  const void* const* b = a->buffers;
  switch (fn->kind) {
    case 0:
      return vpq_affine_qmv_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                       const_cast<void*>(b[4]), a->K, a->N, a->M < 1 ? 1 : a->M,
                                       stream);
    case 1:
      return vpq_affine_qmm_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                       const_cast<void*>(b[4]), a->K, a->N, a->M, stream);
    case 2:
      return vpq_affine_dequant_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2],
                                           const_cast<void*>(b[3]), a->K, a->N, stream);
    case 3:
    case 4:
      return vpq_affine_quant_w4_g64(b[0], fn->kind == 3 ? 1 : 0,
                                     static_cast<uint32_t*>(const_cast<void*>(b[1])),
                                     const_cast<void*>(b[2]), const_cast<void*>(b[3]), a->K, a->N,
                                     a->clip, stream);
    case 5:
      return vpq_affine_qmv_w4g64_bf16_add(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                           const_cast<void*>(b[4]), a->K, a->N, a->M < 1 ? 1 : a->M, b[7],
                                           stream);
    case 6:
      return vpq_affine_qmv_swiglu_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                              const_cast<void*>(b[4]), a->K, a->N, a->M < 1 ? 1 : a->M, stream);
    case 7:
      return vpq_affine_qmv_qkv_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                           const_cast<void*>(b[4]), const_cast<void*>(b[5]),
                                           const_cast<void*>(b[6]), a->K, a->q_rows, a->k_rows, a->v_rows,
                                           a->M < 1 ? 1 : a->M, stream);
    case 8:
      return vpq_affine_qmm_swiglu_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                              const_cast<void*>(b[4]), a->K, a->N, a->M, stream);
    case 9:
      return vpq_affine_qmv_batch_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                             const_cast<void*>(b[4]), a->K, a->N, a->M < 1 ? 1 : a->M, stream);
    case 72:
      return vpq_affine_qmm_grouped_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                               const_cast<void*>(b[4]), a->K, a->N, a->M, static_cast<const int*>(b[8]),
                                               static_cast<const int*>(b[9]), a->experts, a->rows, stream);
    case 73:
      return vpq_affine_qmm_grouped_swiglu_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                                      const_cast<void*>(b[4]), a->K, a->N, a->M,
                                                      static_cast<const int*>(b[8]), static_cast<const int*>(b[9]),
                                                      a->experts, a->rows, const_cast<void*>(b[10]), stream);
    case 74:
      return vpq_affine_qmm_grouped_geglu_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                                     const_cast<void*>(b[4]), a->K, a->N, a->M,
                                                     static_cast<const int*>(b[8]), static_cast<const int*>(b[9]),
                                                     a->experts, a->rows, const_cast<void*>(b[10]), stream);
    case 97:
      return vpq_affine_qmm_grouped_w8g64_bf16(0, static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                               const_cast<void*>(b[4]), a->K, a->N, a->M, static_cast<const int*>(b[8]),
                                               static_cast<const int*>(b[9]), a->experts, a->rows, nullptr, stream);
    case 98:
    case 99:
      return vpq_affine_qmm_grouped_w8g64_bf16(fn->kind == 98 ? 1 : 2, static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                               const_cast<void*>(b[4]), a->K, a->N, a->M, static_cast<const int*>(b[8]),
                                               static_cast<const int*>(b[9]), a->experts, a->rows,
                                               const_cast<void*>(b[10]), stream);
    case 79:
    case 80:
    case 81:
      return vpq_affine_qmm_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3], const_cast<void*>(b[4]), a->K,
                                 a->N, a->M, fn->kind == 81 ? 8 : 4, 32, fn->kind == 80 ? 2 : 0, stream);
    case 75:
    case 100:
    case 101:
    case 76:
    case 77:
    case 78:
    case 91:
    case 92:
    case 93: {
      vpq_linear_desc d;
      std::memset(&d, 0, sizeof(d));
      d.w = static_cast<const uint32_t*>(b[0]);
      d.scales = b[1];
      d.biases = b[2];
      d.x = b[3];
      d.K = a->K;
      d.M = a->M < 1 ? 1 : a->M;
      if (fn->kind == 75 || fn->kind == 100 || fn->kind == 101) {  // slot 4 = norm_w, 5..7 = q, k, v outputs, eps as a constant
        d.norm_w = b[4];
        d.eps = a->eps;
        d.y = const_cast<void*>(b[5]);
        d.epilogue = VPQ_EPILOGUE_QKV;
        d.aux = b[6];
        d.y3 = const_cast<void*>(b[7]);
        d.q_rows = a->q_rows;
        d.k_rows = a->k_rows;
        d.N = a->q_rows + a->k_rows + a->v_rows;
      } else {               // slot 7 = pair_eid [M]; the gate|up pairs of one token share its x row
        d.y = const_cast<void*>(b[4]);
        d.N = a->N;
        d.expert = static_cast<const int32_t*>(b[7]);
        d.experts = a->experts;
        const int k = fn->kind;
        d.x_div = (k == 78 || k == 93) ? 1 : (int32_t)(a->top_k < 1 ? 1 : a->top_k);
        d.epilogue = (k == 76 || k == 91)   ? VPQ_EPILOGUE_SWIGLU
                     : (k == 77 || k == 92) ? VPQ_EPILOGUE_GEGLU
                                            : VPQ_EPILOGUE_NONE;
      }
      if (fn->kind == 101) { return vpq_affine_qmv_w4g32_bf16_fused(&d, stream); }
      if (fn->kind >= 91) { return vpq_affine_qmv_w8g64_bf16_fused(&d, stream); }  // 91..93, 100: 8-bit
      return vpq_affine_qmv_w4g64_bf16_batch(&d, 1, stream);
    }
    case 70:
    case 71:
      return vpq_affine_qmm_swiglu_bf16_rs(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3], const_cast<void*>(b[4]),
                                           a->K, a->N, a->M, fn->kind == 71 ? 8 : 4, a->out_stride, a->out_off, stream);
    case 82:
    case 83:
    case 84:
    case 85:
    case 86:
    case 87:
    case 88: {  // group-32 GEMVs with a fused store; 86..88 ignore slot 2 (bias = -8 * scale)
      vpq_linear_desc d;
      std::memset(&d, 0, sizeof(d));
      d.w = static_cast<const uint32_t*>(b[0]);
      d.scales = b[1];
      d.biases = b[2];
      d.x = b[3];
      d.y = const_cast<void*>(b[4]);
      d.K = a->K;
      d.M = a->M < 1 ? 1 : a->M;
      d.N = a->N;
      const int k = fn->kind;
      if (k == 85) {
        d.epilogue = VPQ_EPILOGUE_QKV;
        d.aux = b[5];
        d.y3 = const_cast<void*>(b[6]);
        d.q_rows = a->q_rows;
        d.k_rows = a->k_rows;
        d.N = a->q_rows + a->k_rows + a->v_rows;
      } else if (k == 82 || k == 87) {
        d.epilogue = VPQ_EPILOGUE_ADD;
        d.aux = b[7];
      } else if (k == 83 || k == 88) {
        d.epilogue = VPQ_EPILOGUE_GEGLU;
      } else if (k == 84) {
        d.epilogue = VPQ_EPILOGUE_GELU_MUL;
        d.aux = b[7];
      }
      return k >= 86 ? vpq_affine_qmv_w4g32_q40_bf16_fused(&d, stream) : vpq_affine_qmv_w4g32_bf16_fused(&d, stream);
    }
    case 107:
    case 108: {
      vpq_linear_desc d;
      std::memset(&d, 0, sizeof(d));
      d.w = static_cast<const uint32_t*>(b[0]);
      d.scales = b[1];
      d.biases = b[2];
      d.x = b[3];
      d.y = const_cast<void*>(b[4]);
      d.K = a->K;
      d.N = a->N;
      d.M = a->M < 1 ? 1 : a->M;
      d.epilogue = fn->kind == 107 ? VPQ_EPILOGUE_SWIGLU : VPQ_EPILOGUE_GEGLU;
      return vpq_affine_qmv_batch_w4g64_bf16_fused(&d, stream);
    }
    case 103:
    case 104:
    case 105:
    case 106: {
      // sorted slots in tiles of two (slot 7 = srow [M], 8 = tile2e [M / 2]); gate|up gathers its x rows
      // through srow, down reads the sorted activations by slot; dead slots are not written
      vpq_linear_desc d;
      std::memset(&d, 0, sizeof(d));
      d.w = static_cast<const uint32_t*>(b[0]);
      d.scales = b[1];
      d.biases = b[2];
      d.x = b[3];
      d.y = const_cast<void*>(b[4]);
      d.K = a->K;
      d.N = a->N;
      d.M = a->M < 1 ? 1 : a->M;
      d.row_map = static_cast<const int32_t*>(b[7]);
      d.expert = static_cast<const int32_t*>(b[8]);
      d.experts = a->experts;
      d.expert_div = 2;
      const bool gate_up = fn->kind == 103 || fn->kind == 105;
      d.row_gather = gate_up ? 1 : 0;
      d.epilogue = gate_up ? VPQ_EPILOGUE_SWIGLU : VPQ_EPILOGUE_NONE;
      return fn->kind >= 105 ? vpq_affine_qmv_w8g64_bf16_fused(&d, stream) : vpq_affine_qmv_w4g64_bf16_batch(&d, 1, stream);
    }
    case 95:
    case 96: {
      // Separate gate and up matrices of different widths (slots: gate 0..2, up 3..5, x 6, y 7, pair_eid 10;
      // N = ffn): the up GEMV writes y, the gate GEMV multiplies silu(gate) into it.
      vpq_linear_desc up, gate;
      std::memset(&up, 0, sizeof(up));
      up.w = static_cast<const uint32_t*>(b[3]);
      up.scales = b[4];
      up.biases = b[5];
      up.x = b[6];
      up.y = const_cast<void*>(b[7]);
      up.K = a->K;
      up.N = a->N;
      up.M = a->M < 1 ? 1 : a->M;
      up.expert = static_cast<const int32_t*>(b[10]);
      up.experts = a->experts;
      up.x_div = (int32_t)(a->top_k < 1 ? 1 : a->top_k);
      gate = up;
      gate.w = static_cast<const uint32_t*>(b[0]);
      gate.scales = b[1];
      gate.biases = b[2];
      gate.epilogue = VPQ_EPILOGUE_SILU_MUL;
      gate.aux = b[7];
      const bool gate_w4 = fn->kind == 95;
      if (int rc = gate_w4 ? vpq_affine_qmv_w8g64_bf16_fused(&up, stream) : vpq_affine_qmv_w4g64_bf16_batch(&up, 1, stream)) {
        return rc;
      }
      return gate_w4 ? vpq_affine_qmv_w4g64_bf16_batch(&gate, 1, stream) : vpq_affine_qmv_w8g64_bf16_fused(&gate, stream);
    }
    case 94:
      return vpq_affine_moe_gate_w8g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3], const_cast<void*>(b[4]),
                                            a->K, a->M < 1 ? 1 : a->M, stream);
    case 89:
      return vpq_affine_requant_w8_to_w4_g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2],
                                                  static_cast<uint32_t*>(const_cast<void*>(b[3])), const_cast<void*>(b[4]),
                                                  const_cast<void*>(b[5]), a->K, a->N, stream);
    case 66:
    case 67:
    case 68:
    case 69:
    case 90:
    case 102: {
      vpq_linear_desc d;
      std::memset(&d, 0, sizeof(d));
      d.w = static_cast<const uint32_t*>(b[0]);
      d.scales = b[1];
      d.biases = b[2];
      d.x = b[3];
      d.y = const_cast<void*>(b[4]);
      d.K = a->K;
      d.M = a->M < 1 ? 1 : a->M;
      if (fn->kind == 68) {  // slots 4..6 = q, k, v outputs; the row counts give N
        d.epilogue = VPQ_EPILOGUE_QKV;
        d.aux = b[5];
        d.y3 = const_cast<void*>(b[6]);
        d.q_rows = a->q_rows;
        d.k_rows = a->k_rows;
        d.N = a->q_rows + a->k_rows + a->v_rows;
      } else if (fn->kind == 102) {
        d.N = a->N;
        return vpq_affine_qmv_w8g32_bf16_fused(&d, stream);
      } else {
        d.epilogue = fn->kind == 66   ? VPQ_EPILOGUE_ADD
                     : fn->kind == 67 ? VPQ_EPILOGUE_SWIGLU
                     : fn->kind == 90 ? VPQ_EPILOGUE_GEGLU
                                      : VPQ_EPILOGUE_GELU_MUL;
        d.aux = (fn->kind == 67 || fn->kind == 90) ? nullptr : b[7];
        d.N = a->N;
      }
      return vpq_affine_qmv_w8g64_bf16_fused(&d, stream);
    }
    case 61:
      return vpq_affine_qmv_geglu_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                             const_cast<void*>(b[4]), a->K, a->N, a->M < 1 ? 1 : a->M, stream);
    case 62:
      return vpq_affine_qmv_gelu_mul_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                                const_cast<void*>(b[4]), a->K, a->N, a->M < 1 ? 1 : a->M, b[7],
                                                stream);
    case 63:
      return vpq_affine_qmm_geglu_w4g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                             const_cast<void*>(b[4]), a->K, a->N, a->M, stream);
    case 64:
      return vpq_affine_qmm_swiglu_w8g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                              const_cast<void*>(b[4]), a->K, a->N, a->M, stream);
    case 65:
      return vpq_affine_qmm_geglu_w8g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3],
                                             const_cast<void*>(b[4]), a->K, a->N, a->M, stream);
    case 60:
      return vpq_affine_qmv_w4g32_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3], const_cast<void*>(b[4]),
                                       a->K, a->N, a->M < 1 ? 1 : a->M, stream);
    case 59:
      return vpq_affine_qmm_w8g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3], const_cast<void*>(b[4]),
                                       a->K, a->N, a->M, stream);
    case 58:
      return vpq_affine_qmv_w8g64_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], b[3], const_cast<void*>(b[4]),
                                       a->K, a->N, a->M < 1 ? 1 : a->M, stream);
    default: {
      if (fn->kind < 10 || fn->kind >= 10 + 48) { return fail(VPQ_ERR_NOT_FOUND, "dispatch: corrupt function handle"); }
      const int code = fn->kind - 10, quant = code >> 4, bits = (code & 4) ? 8 : 4, group = (code & 1) ? 32 : 64;
      if (quant) {
        return vpq_affine_quant(b[0], quant == 2 ? 1 : 0, static_cast<uint32_t*>(const_cast<void*>(b[1])),
                                const_cast<void*>(b[2]), const_cast<void*>(b[3]), a->K, a->N, bits, group, a->clip,
                                stream);
      }
      return vpq_affine_dequant_bf16(static_cast<const uint32_t*>(b[0]), b[1], b[2], const_cast<void*>(b[3]), a->K,
                                     a->N, bits, group, stream);
    }
  }
}
