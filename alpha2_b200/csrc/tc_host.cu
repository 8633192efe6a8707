// Host side of the tensor-core kernels: tensor-map encoding (through the driver entry
// point, so the library does not link libcuda) and the device error word that the bounded
// waits report into.
#include <mutex>

#include "tc_common.cuh"

namespace alpha {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
    else
      cudaGetLastError();
  });
  return fn;
}

int encode_tmap_2d_bf16(CUtensorMap *out, const void *base, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                        uint32_t box_inner, uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return set_error("tensor map: cuTensorMapEncodeTiled is not available from this driver");
  if (((uintptr_t)base & 15) != 0) return set_error("tensor map: base address %p is not 16-byte aligned", base);
  if ((ld_elems * 2) % 16 != 0)
    return set_error("tensor map: leading dimension %llu (bf16 elements) must be a multiple of 8",
                     (unsigned long long)ld_elems);
  if (box_inner * 2 != 128) return set_error("tensor map: inner box must be 64 bf16 (128-byte swizzle)");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error("cuTensorMapEncodeTiled failed (%d): dims %llu x %llu, ld %llu, box %u x %u", (int)r,
                     (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)ld_elems, box_inner,
                     box_outer);
  return 0;
}

int encode_tmap_2d_out(CUtensorMap *out, const void *base, int dtype, uint64_t inner, uint64_t outer, uint64_t ld_elems,
                       uint32_t box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return set_error("tensor map: cuTensorMapEncodeTiled is not available from this driver");
  const uint64_t es = dtype == ALPHA_F32 ? 4 : 2;
  if (((uintptr_t)base & 15) != 0 || (ld_elems * es) % 16 != 0)
    return set_error("tensor map: output base / leading dimension not 16-byte aligned");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * es};
  cuuint32_t box[2] = {(cuuint32_t)(128 / es), box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dtype == ALPHA_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error("cuTensorMapEncodeTiled (output) failed (%d)", (int)r);
  return 0;
}

int encode_tmap_3d_bf16(CUtensorMap *out, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t ld1_elems,
                        uint64_t ld2_elems, uint32_t box0, uint32_t box1, uint32_t box2) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return set_error("tensor map: cuTensorMapEncodeTiled is not available from this driver");
  if (((uintptr_t)base & 15) != 0) return set_error("tensor map: base address %p is not 16-byte aligned", base);
  if ((ld1_elems * 2) % 16 != 0 || (ld2_elems * 2) % 16 != 0)
    return set_error("tensor map: strides %llu / %llu (bf16 elements) must be multiples of 8",
                     (unsigned long long)ld1_elems, (unsigned long long)ld2_elems);
  if (box0 * 2 != 128) return set_error("tensor map: inner box must be 64 bf16 (128-byte swizzle)");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1_elems * 2, ld2_elems * 2};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error("cuTensorMapEncodeTiled (3d) failed (%d)", (int)r);
  return 0;
}

int encode_tmap_4d_bf16(CUtensorMap *out, const void *base, uint64_t D, uint64_t T, uint64_t H, uint64_t Bn,
                        uint64_t st, uint64_t sh, uint64_t sb, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return set_error("tensor map: cuTensorMapEncodeTiled is not available from this driver");
  if (((uintptr_t)base & 15) != 0) return set_error("tensor map: base address %p is not 16-byte aligned", base);
  if (D != 64) return set_error("tensor map: attention head dim must be 64 (one 128-byte swizzle row)");
  // a dimension of extent 1 still needs a legal stride
  if (H == 1 && (sh == 0 || (sh * 2) % 16 != 0)) sh = st * T;
  if (Bn == 1 && (sb == 0 || (sb * 2) % 16 != 0)) sb = st * T;
  if ((st * 2) % 16 != 0 || (sh * 2) % 16 != 0 || (sb * 2) % 16 != 0 || sh == 0 || sb == 0)
    return set_error("tensor map: attention strides (%llu, %llu, %llu) must be non-zero multiples of 8 elements",
                     (unsigned long long)st, (unsigned long long)sh, (unsigned long long)sb);
  cuuint64_t dims[4] = {D, T, H, Bn};
  cuuint64_t strides[3] = {st * 2, sh * 2, sb * 2};
  cuuint32_t box[4] = {64, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error("cuTensorMapEncodeTiled (4d) failed (%d): T=%llu H=%llu B=%llu strides %llu/%llu/%llu", (int)r,
                     (unsigned long long)T, (unsigned long long)H, (unsigned long long)Bn, (unsigned long long)st,
                     (unsigned long long)sh, (unsigned long long)sb);
  return 0;
}

static uint32_t *g_err_word = nullptr;

uint32_t *tc_error_word() {
  if (!g_err_word) {
    if (cudaMalloc(&g_err_word, sizeof(uint32_t)) != cudaSuccess) {
      cudaGetLastError();
      g_err_word = nullptr;
      return nullptr;
    }
    cudaMemsetAsync(g_err_word, 0, sizeof(uint32_t), g_stream);
  }
  return g_err_word;
}

// Shutdown: the word belongs to the device that is being left.
void tc_error_word_free() {
  if (g_err_word) cudaFree(g_err_word);
  g_err_word = nullptr;
}

int tc_check_error(const char *who) {
  if (!g_err_word) return 0;
  uint32_t v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, g_err_word, sizeof(v), cudaMemcpyDeviceToHost, g_stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(g_stream);
  if (e != cudaSuccess) return set_error("%s: %s", who, cudaGetErrorString(e));
  if (v != 0) {
    cudaMemsetAsync(g_err_word, 0, sizeof(uint32_t), g_stream);
    return set_error("%s: a tensor-core kernel gave up a bounded wait (code 0x%x); its output is invalid", who, v);
  }
  return 0;
}

}  // namespace tc
}  // namespace alpha

// Waits for all enqueued work and reports whether any tensor-core kernel abandoned a
// bounded wait since the last check.
extern "C" int alpha_check_async_error(void) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CUDA(cudaStreamSynchronize(alpha::g_stream));
  return alpha::tc::tc_check_error("alpha_check_async_error");
}
