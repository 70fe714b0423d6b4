// TVM-FFI module exporting the reference's own FFI symbol for this path,
//   fast_topk(score, indices, lengths, row_starts, has_row_starts)
// (jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:1285-1290 and :1387), so that the reference's
// unmodified Python wrapper (jit_kernel/topk_indexer.py:137-151) runs on this library when its
// module loader returns this module instead of JIT-compiling its own source.
//
// Host code only: it unpacks the DLPack views and forwards to the C ABI of libff_topk.so
// (include/ff_topk.h) on the stream tvm_ffi reports as current, as the reference does
// (topk_indexer_radix.cu:1304-1307).  Differences from the reference symbol: any topk in
// [1, 2048] is accepted (the reference throws unless it is 512, 1024 or 2048), the indices come
// back in canonical order, and every output slot is written.
//
// The reference's signature carries no scratch buffer.  Batches of up to FF_TOPK_STATIC_MAX_ROWS
// rows go through ff_topk_launch_static, whose scratch is built into the library, so that long
// rows are still split over the whole GPU; like that entry point, two such calls must not overlap
// on one GPU.  Larger batches need no scratch (every row stays inside one cluster).
#include <tvm/ffi/container/tensor.h>
#include <tvm/ffi/extra/c_env_api.h>
#include <tvm/ffi/function.h>

#include <stdexcept>
#include <string>

#include "../../include/ff_topk.h"

namespace {

void require(bool cond, const char* what) {
  if (!cond) throw std::runtime_error(std::string("fast_topk: ") + what);
}

bool is_dtype(const tvm::ffi::TensorView& t, int code, int bits) {
  const DLDataType d = t.dtype();
  return d.code == code && d.bits == bits && d.lanes == 1;
}

void ff_fast_topk(tvm::ffi::TensorView score, tvm::ffi::TensorView indices, tvm::ffi::TensorView lengths,
                  tvm::ffi::TensorView row_starts, int64_t has_row_starts) {
  require(score.ndim() == 2 && indices.ndim() == 2 && lengths.ndim() == 1, "score and indices must be 2-D, lengths 1-D");
  require(is_dtype(score, kDLFloat, 32), "score must be float32");
  require(is_dtype(indices, kDLInt, 32) && is_dtype(lengths, kDLInt, 32), "indices and lengths must be int32");
  const int64_t B = score.size(0), L = score.size(1), topk = indices.size(1);
  require(indices.size(0) == B && lengths.size(0) == B, "indices and lengths must have one row per score row");
  require(L == 0 || score.stride(1) == 1, "score.stride(1) must be 1");
  require(B == 0 || topk == 0 || (indices.stride(1) == 1 && indices.stride(0) == topk), "indices must be contiguous");
  require(B <= 1 || lengths.stride(0) == 1, "lengths must be contiguous");
  const int32_t* rs = nullptr;
  if (has_row_starts != 0) {
    require(row_starts.ndim() == 1 && row_starts.size(0) == B && is_dtype(row_starts, kDLInt, 32) &&
                (B <= 1 || row_starts.stride(0) == 1),
            "row_starts must be a contiguous int32 [B] tensor");
    rs = static_cast<const int32_t*>(row_starts.data_ptr());
  }
  const DLDevice dev = score.device();
  require(dev.device_type == kDLCUDA, "score must live on a CUDA device (there is no CPU path)");
  void* stream = TVMFFIEnvGetStream(dev.device_type, dev.device_id);
  const int64_t row_stride = B > 1 ? score.stride(0) : (score.stride(0) > L ? score.stride(0) : L);
  int rc;
  if (B <= FF_TOPK_STATIC_MAX_ROWS) {
    rc = ff_topk_launch_static(static_cast<const float*>(score.data_ptr()), row_stride,
                               static_cast<const int32_t*>(lengths.data_ptr()), rs,
                               static_cast<int32_t*>(indices.data_ptr()), static_cast<int32_t>(B), L,
                               static_cast<int32_t>(topk), nullptr, stream);
  } else {
    rc = ff_topk_launch(static_cast<const float*>(score.data_ptr()), row_stride,
                        static_cast<const int32_t*>(lengths.data_ptr()), rs, static_cast<int32_t*>(indices.data_ptr()),
                        static_cast<int32_t>(B), L, static_cast<int32_t>(topk), nullptr, 0, nullptr, stream);
  }
  if (rc != 0) throw std::runtime_error(std::string("fast_topk: ") + ff_last_error_string());
}

}  // namespace

TVM_FFI_DLL_EXPORT_TYPED_FUNC(fast_topk, ff_fast_topk);
