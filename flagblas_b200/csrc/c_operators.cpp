// pybind11 module `flagblas_b200.c_operators`: a thin, torch-free binding of the C ABI declared in
// include/flagblas_b200.h.  The reference reserves exactly this module name for a compiled back end
// (`from flag_blas import c_operators`, src/flag_blas/config.py:35-41).  Every function takes raw
// addresses as Python ints, forwards to the matching extern "C" entry point and returns its status.
#include <pybind11/pybind11.h>

#include <cstdint>

#include "../../include/flagblas_b200.h"

namespace py = pybind11;
using addr = std::uintptr_t;

static inline void* p(addr a) { return reinterpret_cast<void*>(a); }
template <class T> static inline const T* cp(addr a) { return reinterpret_cast<const T*>(a); }

PYBIND11_MODULE(c_operators, m) {
  m.doc() = "flagblas_b200 C-ABI binding (sm_100a GEMM back end)";
  m.def("gemm", [](int dtype, int ta, int tb, int64_t mm, int64_t nn, int64_t kk, float alpha, addr a, int64_t lda, addr b,
                   int64_t ldb, float beta, addr c, int64_t ldc, addr ws, size_t ws_bytes, addr stream) {
    return fb_gemm(dtype, ta, tb, mm, nn, kk, alpha, p(a), lda, p(b), ldb, beta, p(c), ldc, p(ws), ws_bytes, p(stream));
  });
  m.def("gemm_workspace_bytes", [](int dtype, int ta, int tb, int64_t mm, int64_t nn, int64_t kk, addr a, int64_t lda, addr b,
                                   int64_t ldb) { return fb_gemm_workspace_bytes(dtype, ta, tb, mm, nn, kk, p(a), lda, p(b), ldb); });
  m.def("gemm_ex", [](int dtype, int ta, int tb, int64_t mm, int64_t nn, int64_t kk, double alpha_re, double alpha_im, addr a,
                      int64_t lda, addr b, int64_t ldb, double beta_re, double beta_im, addr c, int64_t ldc, addr stream) {
    const double alpha[2] = {alpha_re, alpha_im}, beta[2] = {beta_re, beta_im};
    return fb_gemm_ex(dtype, ta, tb, mm, nn, kk, alpha, p(a), lda, p(b), ldb, beta, p(c), ldc, p(stream));
  });
  m.def("trmm", [](int dtype, int side, int uplo, int trans, int diag, int64_t mm, int64_t nn, double alpha_re, double alpha_im,
                   addr a, int64_t lda, addr b, int64_t ldb, addr c, int64_t ldc, addr stream) {
    const double alpha[2] = {alpha_re, alpha_im};
    return fb_trmm(dtype, side, uplo, trans, diag, mm, nn, alpha, p(a), lda, p(b), ldb, p(c), ldc, p(stream));
  });
  m.def("gemv", [](int dtype, int trans, int64_t mm, int64_t nn, float alpha, addr a, int64_t lda, addr x, int64_t incx,
                   float beta, addr y, int64_t incy, addr ws, size_t ws_bytes, addr stream) {
    return fb_gemv(dtype, trans, mm, nn, alpha, p(a), lda, p(x), incx, beta, p(y), incy, p(ws), ws_bytes, p(stream));
  });
  m.def("gemv_workspace_bytes",
        [](int dtype, int trans, int64_t mm, int64_t nn) { return fb_gemv_workspace_bytes(dtype, trans, mm, nn); });
  m.def("gemv_fp8", [](int a_fmt, int x_fmt, int y_dtype, int64_t mm, int64_t nn, float alpha, addr a, int64_t lda, addr x,
                       int64_t incx, float beta, addr y, int64_t incy, addr ws, size_t ws_bytes, addr stream) {
    return fb_gemv_fp8(a_fmt, x_fmt, y_dtype, mm, nn, alpha, p(a), lda, p(x), incx, beta, p(y), incy, p(ws), ws_bytes, p(stream));
  });
  m.def("gemv_fp8_workspace_bytes", [](int64_t mm, int64_t nn) { return fb_gemv_fp8_workspace_bytes(mm, nn); });
  m.def("group_gemm", [](int dtype, int b_k_contig, addr da, addr db, addr dc, addr dout, addr dm, addr dn, addr dk, addr dlda,
                         addr dldb, addr dldc, int groups, int64_t mh, int64_t nh, int64_t kh, float alpha, float beta, addr ws,
                         size_t ws_bytes, addr stream) {
    return fb_group_gemm(dtype, b_k_contig, cp<int64_t>(da), cp<int64_t>(db), cp<int64_t>(dc), cp<int64_t>(dout), cp<int32_t>(dm),
                         cp<int32_t>(dn), cp<int32_t>(dk), cp<int32_t>(dlda), cp<int32_t>(dldb), cp<int32_t>(dldc), groups, mh, nh,
                         kh, alpha, beta, p(ws), ws_bytes, p(stream));
  });
  m.def("group_gemm_prepare", [](int dtype, int b_k_contig, addr da, addr db, addr dc, addr dout, addr dm, addr dn, addr dk,
                                 addr dlda, addr dldb, addr dldc, int groups, int64_t mh, int64_t nh, int64_t kh, addr ws,
                                 size_t ws_bytes, addr stream) {
    return fb_group_gemm_prepare(dtype, b_k_contig, cp<int64_t>(da), cp<int64_t>(db), cp<int64_t>(dc), cp<int64_t>(dout),
                                 cp<int32_t>(dm), cp<int32_t>(dn), cp<int32_t>(dk), cp<int32_t>(dlda), cp<int32_t>(dldb),
                                 cp<int32_t>(dldc), groups, mh, nh, kh, p(ws), ws_bytes, p(stream));
  });
  m.def("group_gemm_run", [](int dtype, int b_k_contig, int groups, int64_t mh, int64_t nh, int64_t kh, float alpha, float beta,
                             addr ws, size_t ws_bytes, addr stream) {
    return fb_group_gemm_run(dtype, b_k_contig, groups, mh, nh, kh, alpha, beta, p(ws), ws_bytes, p(stream));
  });
  m.def("group_gemm_no_alloc", [](int dtype, int b_k_contig, addr da, addr db, addr dc, addr dout, addr dm, addr dn, addr dk,
                                  addr dlda, addr dldb, addr dldc, int groups, int64_t mh, int64_t nh, int64_t kh, float alpha,
                                  float beta, addr stream) {
    return fb_group_gemm_no_alloc(dtype, b_k_contig, cp<int64_t>(da), cp<int64_t>(db), cp<int64_t>(dc), cp<int64_t>(dout),
                                  cp<int32_t>(dm), cp<int32_t>(dn), cp<int32_t>(dk), cp<int32_t>(dlda), cp<int32_t>(dldb),
                                  cp<int32_t>(dldc), groups, mh, nh, kh, alpha, beta, p(stream));
  });
  m.def("group_mm", [](int dtype, int b_k_contig, addr a, int64_t lda, addr b, int64_t ldb, int64_t b_group_stride, addr c,
                       int64_t ldc, addr offs, int groups, int64_t nn, int64_t kk, addr ws, size_t ws_bytes, addr stream) {
    return fb_group_mm(dtype, b_k_contig, p(a), lda, p(b), ldb, b_group_stride, p(c), ldc, cp<int32_t>(offs), groups, nn, kk, p(ws),
                       ws_bytes, p(stream));
  });
  m.def("group_workspace_bytes", &fb_group_workspace_bytes);
  m.def("no_alloc_max_groups", &fb_no_alloc_max_groups);
  m.def("status_string", [](int s) { return std::string(fb_status_string(s)); });
  m.def("device_status", &fb_device_status);
  m.def("last_cuda_error", &fb_last_cuda_error);
  m.def("sm_count", &fb_sm_count);
  m.def("reload_env", &fb_reload_env);
  m.def("selftest_bounded_wait", [](int64_t limit, addr stream) { return fb_selftest_bounded_wait(limit, p(stream)); });
  m.def("debug_set_profile_buffer", [](addr buf) { fb_debug_set_profile_buffer(p(buf)); });
  m.attr("FB_F32") = static_cast<int>(FB_F32);
  m.attr("FB_TF32") = static_cast<int>(FB_TF32);
  m.attr("FB_F16") = static_cast<int>(FB_F16);
  m.attr("FB_BF16") = static_cast<int>(FB_BF16);
}
