// XLA FFI handler for the sm_100a ragged paged attention: the shim a JAX host registers with
//   jax.ffi.register_ffi_target("ejk_rpa_sm100", jax.ffi.pycapsule(lib.EjkRpaSm100), platform="CUDA")
// and calls with jax.ffi.ffi_call("ejk_rpa_sm100", (out_type, workspace_type, status_type))(...).
//
// SOURCE ONLY: it needs the headers shipped with jaxlib (xla/ffi/api/ffi.h).  Neither jax nor
// jaxlib is installed in the environment this library is built and tested in, so this file is
// not part of the build (the build script compiles csrc/*.cu only) and has never been compiled.
// It documents the exact binding: seven operands, three results (output, scratch, status word),
// scalars as attributes, XLA's stream, no allocation and no host synchronisation -- the same
// shape of boundary as the reference's Triton custom call (ejkernel/callib/_triton_call.py:737-757).
//
// Build (where jaxlib is present):
//   g++ -std=c++17 -fPIC -shared -I$(python -c "import jaxlib, os; print(os.path.join(os.path.dirname(jaxlib.__file__), 'include'))") \
//       -Iinclude ejk_rpa_xla_ffi.cc -L ejkernel_b200/lib -lejk_rpa -o libejk_rpa_ffi.so
#if __has_include("xla/ffi/api/ffi.h")
#include <cuda_runtime_api.h>

#include "ejk_rpa.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

static ffi::Error EjkRpaSm100Impl(cudaStream_t stream, ffi::AnyBuffer queries, ffi::AnyBuffer kv_pages,
                                  ffi::Buffer<ffi::S32> context_lens, ffi::Buffer<ffi::S32> block_tables,
                                  ffi::Buffer<ffi::S32> query_start_loc, ffi::Buffer<ffi::S32> num_seqs,
                                  ffi::Buffer<ffi::F32> softmax_aux,  // shape [rows, 0] when absent
                                  ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::Buffer<ffi::U8>> workspace,
                                  ffi::Result<ffi::Buffer<ffi::S32>> status, float softmax_scale,
                                  float logits_soft_cap, int32_t sliding_window, int32_t num_kv_pages_per_block,
                                  int32_t num_queries_per_block) {
  const auto qd = queries.dimensions();
  const auto kd = kv_pages.dimensions();
  const auto td = block_tables.dimensions();
  if (qd.size() != 3 || kd.size() != 4 || td.size() != 2)
    return ffi::Error::InvalidArgument("ragged_page_attention: wrong operand ranks");
  ejk_rpa_shape shape{};
  shape.total_tokens = static_cast<int32_t>(qd[0]);
  shape.num_q_heads = static_cast<int32_t>(qd[1]);
  shape.head_dim = static_cast<int32_t>(qd[2]);
  shape.num_pages = static_cast<int32_t>(kd[0]);
  shape.page_size = static_cast<int32_t>(kd[1]);
  shape.num_kv_heads = static_cast<int32_t>(kd[2] / 2);
  shape.max_num_seqs = static_cast<int32_t>(td[0]);
  shape.pages_per_seq = static_cast<int32_t>(td[1]);
  switch (queries.element_type()) {
    case ffi::BF16: shape.dtype = EJK_RPA_BF16; break;
    case ffi::F16: shape.dtype = EJK_RPA_F16; break;
    default: return ffi::Error::InvalidArgument("ragged_page_attention[cuda]: bf16 or f16 only");
  }
  // the pool has the queries' dtype, or holds float8 e4m3 bytes
  if (kv_pages.element_type() == ffi::F8E4M3FN) shape.kv_dtype = EJK_RPA_E4M3;
  else if (kv_pages.element_type() != queries.element_type())
    return ffi::Error::InvalidArgument("ragged_page_attention[cuda]: kv_pages must have the queries' dtype or be float8_e4m3fn");
  ejk_rpa_attrs attrs{};
  attrs.softmax_scale = softmax_scale;
  attrs.logits_soft_cap = logits_soft_cap;  // 0 = none
  attrs.sliding_window = sliding_window;    // <= 0 = none
  const auto ad = softmax_aux.dimensions();
  attrs.num_sinks = ad.size() == 2 ? static_cast<int32_t>(ad[1]) : 0;
  attrs.sink_rows = ad.size() == 2 ? static_cast<int32_t>(ad[0]) : 0;
  attrs.num_kv_pages_per_block = num_kv_pages_per_block;  // tile hints of RaggedPageAttentionConfig, 0 = auto
  attrs.num_queries_per_block = num_queries_per_block;
  // the scratch result must be what ejk_rpa_workspace_bytes() asked for: say so here, by name, instead of
  // letting the launch answer with a bare error code
  if (workspace->size_bytes() < ejk_rpa_workspace_bytes_min(&shape) ||
      (reinterpret_cast<uintptr_t>(workspace->typed_data()) & 255))
    return ffi::Error::InvalidArgument(
        "ragged_page_attention[cuda]: the workspace result must hold ejk_rpa_workspace_bytes(shape) bytes, 256-byte aligned");
  // `out` is a fresh, uninitialised XLA buffer: the launch itself writes every row of it (rows past the last
  // sequence are zero-filled by the kernels), so no memset is needed here
  // the status word is a fresh result buffer: clear it on the stream before the kernels OR bits in
  cudaMemsetAsync(status->typed_data(), 0, sizeof(int32_t), stream);
  const int rc = ejk_rpa_launch(queries.untyped_data(), kv_pages.untyped_data(), context_lens.typed_data(),
                                block_tables.typed_data(), query_start_loc.typed_data(), num_seqs.typed_data(),
                                attrs.num_sinks ? softmax_aux.typed_data() : nullptr, out->untyped_data(),
                                workspace->typed_data(), workspace->size_bytes(), status->typed_data(), &shape, &attrs,
                                stream);
  if (rc != 0) return ffi::Error::Internal(ejk_rpa_error_string(rc));
  return ffi::Error::Success();
}

XLA_FFI_DEFINE_HANDLER_SYMBOL(EjkRpaSm100, EjkRpaSm100Impl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()           // queries
                                  .Arg<ffi::AnyBuffer>()           // kv_pages
                                  .Arg<ffi::Buffer<ffi::S32>>()    // context_lens
                                  .Arg<ffi::Buffer<ffi::S32>>()    // block_tables
                                  .Arg<ffi::Buffer<ffi::S32>>()    // query_start_loc
                                  .Arg<ffi::Buffer<ffi::S32>>()    // num_seqs
                                  .Arg<ffi::Buffer<ffi::F32>>()    // softmax_aux
                                  .Ret<ffi::AnyBuffer>()           // out
                                  .Ret<ffi::Buffer<ffi::U8>>()     // workspace (ejk_rpa_workspace_bytes)
                                  .Ret<ffi::Buffer<ffi::S32>>()    // status word
                                  .Attr<float>("softmax_scale")
                                  .Attr<float>("logits_soft_cap")
                                  .Attr<int32_t>("sliding_window")
                                  .Attr<int32_t>("num_kv_pages_per_block")
                                  .Attr<int32_t>("num_queries_per_block"));
#endif  // xla/ffi/api/ffi.h available
