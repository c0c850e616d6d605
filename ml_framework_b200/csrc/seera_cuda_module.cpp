// Python module `seera_cuda`: a thin pybind11 shim over the C ABI in include/seera_b200.h.
//
// Exports the same function names, positional argument orders and pointer convention as the
// reference's binding (engine_cuda/src/cuda_bindings.cpp:14-533): device addresses cross as Python
// ints, `dimarr` of the reductions is a host int32 NumPy array, cuda_ones_f / cuda_zeros_f allocate
// and return an address, to_host_* take (address, shape tuple).  A non-zero status from the C ABI
// becomes a RuntimeError carrying seera_last_error(); the reference ignores errors.
// No compute happens here.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <utility>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "seera_b200.h"

namespace py = pybind11;
using arr_f = py::array_t<float, py::array::c_style | py::array::forcecast>;
using arr_i = py::array_t<int32_t, py::array::c_style | py::array::forcecast>;
using arr_s = py::array_t<int16_t, py::array::c_style | py::array::forcecast>;
using uptr = uintptr_t;

static inline void ck(int status) {
    if (status) throw std::runtime_error(std::string("[seera_cuda] ") + seera_last_error());
}
static inline uptr ckp(void *p) {
    if (!p) throw std::runtime_error(std::string("[seera_cuda] ") + seera_last_error());
    return reinterpret_cast<uptr>(p);
}
template <class T> static inline T *P(uptr a) { return reinterpret_cast<T *>(a); }
using F = float;

template <class T, class Arr>
static Arr download(uptr ptr, const py::tuple &shape) {
    std::vector<py::ssize_t> dims;
    size_t n = 1;
    for (auto s : shape) { py::ssize_t d = s.cast<py::ssize_t>(); dims.push_back(d); n *= (size_t)d; }
    Arr out(dims);
    if (n) ck(seera_to_host(out.mutable_data(), P<const void>(ptr), n * sizeof(T)));
    return out;
}

PYBIND11_MODULE(seera_cuda, m) {
    m.doc() = "Seera CUDA engine for NVIDIA B200 (sm_100a)";

    // ---- memory ----------------------------------------------------------------------------------
    m.def("cuda_malloc", [](size_t n) { return ckp(seera_cuda_malloc(n)); });
    m.def("cuda_malloc_f16", [](int n) { return ckp(seera_cuda_malloc_f32(n)); });   // fp32 storage, as in the reference
    m.def("cuda_malloc_f32", [](int n) { return ckp(seera_cuda_malloc_f32(n)); });
    m.def("cuda_malloc_i32", [](int n) { return ckp(seera_cuda_malloc_i32(n)); });
    m.def("cuda_malloc_i16", [](int n) { return ckp(seera_cuda_malloc_i16(n)); });
    m.def("cuda_free", [](uptr p) { seera_cuda_free(P<void>(p)); });
    m.def("cuda_memcopy_devicetodevice", [](uptr d, uptr s, int n) { ck(seera_cuda_memcopy_devicetodevice(P<void>(d), P<const void>(s), n)); });
    m.def("cuda_memset", [](uptr p, int v, size_t n) { ck(seera_cuda_memset(P<void>(p), v, n)); });

    // ---- transfers -------------------------------------------------------------------------------
    m.def("to_device_f16", [](arr_f a) { return ckp(seera_to_device(a.data(), (size_t)a.size() * 4)); });
    m.def("to_device_f32", [](arr_f a) { return ckp(seera_to_device(a.data(), (size_t)a.size() * 4)); });
    m.def("to_device_i32", [](arr_i a) { return ckp(seera_to_device(a.data(), (size_t)a.size() * 4)); });
    m.def("to_device_i16", [](arr_s a) { return ckp(seera_to_device(a.data(), (size_t)a.size() * 2)); });
    m.def("to_host_f16", [](uptr p, py::tuple s) { return download<float, arr_f>(p, s); });
    m.def("to_host_f32", [](uptr p, py::tuple s) { return download<float, arr_f>(p, s); });
    m.def("to_host_i32", [](uptr p, py::tuple s) { return download<int32_t, arr_i>(p, s); });
    m.def("to_host_i16", [](uptr p, py::tuple s) { return download<int16_t, arr_s>(p, s); });

    // ---- unary ops -------------------------------------------------------------------------------
    m.def("cuda_relu_fwd", [](uptr x, uptr o, uptr g, int n) { ck(seera_cuda_relu_fwd(P<const F>(x), P<F>(o), P<F>(g), n)); });
    m.def("cuda_sigmoid_fwd", [](uptr x, uptr o, uptr g, int n) { ck(seera_cuda_sigmoid_fwd(P<const F>(x), P<F>(o), P<F>(g), n)); });
    m.def("cuda_tanh_fwd", [](uptr x, uptr o, uptr g, int n) { ck(seera_cuda_tanh_fwd(P<const F>(x), P<F>(o), P<F>(g), n)); });
    m.def("cuda_log_fwd", [](uptr x, uptr o, uptr g, int n) { ck(seera_cuda_log_fwd(P<const F>(x), P<F>(o), P<F>(g), n)); });
    m.def("cuda_exp_fwd", [](uptr x, uptr o, uptr g, int n) { ck(seera_cuda_exp_fwd(P<const F>(x), P<F>(o), P<F>(g), n)); });
    m.def("cuda_abs_fwd", [](uptr x, uptr o, uptr g, int n) { ck(seera_cuda_abs_fwd(P<const F>(x), P<F>(o), P<F>(g), n)); });
    m.def("cuda_sqrt_fwd", [](uptr x, uptr o, uptr g, int n) { ck(seera_cuda_sqrt_fwd(P<const F>(x), P<F>(o), P<F>(g), n)); });
    m.def("cuda_pow_fwd", [](uptr x, float e, uptr o, uptr g, int n) { ck(seera_cuda_pow_fwd(P<const F>(x), e, P<F>(o), P<F>(g), n)); });
    m.def("cuda_clip_fwd", [](uptr x, float lo, float hi, uptr o, uptr g, int n) { ck(seera_cuda_clip_fwd(P<const F>(x), lo, hi, P<F>(o), P<F>(g), n)); });

    // ---- softmax ---------------------------------------------------------------------------------
    m.def("cuda_softmax_fwd", [](uptr x, uptr o, int N, int C) { ck(seera_cuda_softmax_fwd(P<const F>(x), P<F>(o), N, C)); });
    m.def("cuda_softmax_vjp", [](uptr s, uptr d, uptr dx, int N, int C) { ck(seera_cuda_softmax_vjp(P<const F>(s), P<const F>(d), P<F>(dx), N, C)); });

    // ---- GEMM ------------------------------------------------------------------------------------
    m.def("cuda_matmul", [](uptr A, uptr B, uptr C, int M, int N, int K, int nb) { ck(seera_cuda_matmul(P<const F>(A), P<const F>(B), P<F>(C), M, N, K, nb)); });
    m.def("cuda_matmul_bwd", [](uptr A, uptr B, uptr dC, uptr dA, uptr dB, int M, int N, int K, int nb) {
        ck(seera_cuda_matmul_bwd(P<const F>(A), P<const F>(B), P<const F>(dC), P<F>(dA), P<F>(dB), M, N, K, nb)); });
    m.def("cuda_transpose_2d", [](uptr i, uptr o, int r, int c) { ck(seera_cuda_transpose_2d(P<const F>(i), P<F>(o), r, c)); });
    m.def("cuda_transpose_3d", [](uptr i, uptr o, int nb, int M, int K) { ck(seera_cuda_transpose_3d(P<const F>(i), P<F>(o), nb, M, K)); });

    // ---- convolutions ----------------------------------------------------------------------------
    m.def("cuda_conv2d_fwd", [](uptr x, uptr w, uptr o, int n, int C, int H, int W, int Fo, int R, int S, int ph, int pw, int sh, int sw) {
        ck(seera_cuda_conv2d_fwd(P<const F>(x), P<const F>(w), P<F>(o), n, C, H, W, Fo, R, S, ph, pw, sh, sw)); });
    m.def("cuda_conv2d_bwd", [](uptr w, uptr x, uptr dy, uptr dx, uptr dw, int n, int C, int H, int W, int Fo, int R, int S, int sh, int sw, int ph, int pw) {
        ck(seera_cuda_conv2d_bwd(P<const F>(w), P<const F>(x), P<const F>(dy), P<F>(dx), P<F>(dw), n, C, H, W, Fo, R, S, sh, sw, ph, pw)); });
    m.def("cuda_conv2DTranpose_fwd", [](uptr x, uptr w, uptr o, int n, int Ci, int H, int W, int Co, int KH, int KW, int sh, int sw, int ph, int pw) {
        ck(seera_cuda_conv2DTranpose_fwd(P<const F>(x), P<const F>(w), P<F>(o), n, Ci, H, W, Co, KH, KW, sh, sw, ph, pw)); });
    m.def("cuda_conv2DTranspose_bwd", [](uptr w, uptr x, uptr dy, uptr dx, uptr dw, int n, int Ci, int H, int W, int Co, int KH, int KW, int sh, int sw, int ph, int pw) {
        ck(seera_cuda_conv2DTranspose_bwd(P<const F>(w), P<const F>(x), P<const F>(dy), P<F>(dx), P<F>(dw), n, Ci, H, W, Co, KH, KW, sh, sw, ph, pw)); });

    // ---- pooling ---------------------------------------------------------------------------------
    m.def("cuda_maxpool_fwd", [](uptr x, uptr o, uptr mk, int n, int C, int H, int W, int R, int S, int ph, int pw, int sh, int sw) {
        ck(seera_cuda_maxpool_fwd(P<const F>(x), P<F>(o), P<int>(mk), n, C, H, W, R, S, ph, pw, sh, sw)); });
    m.def("cuda_maxpool_bwd", [](uptr d, uptr mk, uptr dx, int n, int C, int H, int W, int R, int S, int ph, int pw, int sh, int sw) {
        ck(seera_cuda_maxpool_bwd(P<const F>(d), P<const int>(mk), P<F>(dx), n, C, H, W, R, S, ph, pw, sh, sw)); });
    m.def("cuda_unpooling_fwd", [](uptr i, uptr o, int n, int C, int H, int W, int sh, int sw) { ck(seera_cuda_unpooling_fwd(P<const F>(i), P<F>(o), n, C, H, W, sh, sw)); });
    m.def("cuda_unpooling_bwd", [](uptr d, uptr dx, int n, int C, int H, int W, int sh, int sw) { ck(seera_cuda_unpooling_bwd(P<const F>(d), P<F>(dx), n, C, H, W, sh, sw)); });

    // ---- reductions (dimarr: host int32 array) -----------------------------------------------------
    m.def("cuda_sum_fwd", [](uptr A, uptr o, int nd, int dim, arr_i da) { ck(seera_cuda_sum_fwd(P<const F>(A), P<F>(o), nd, dim, da.data())); });
    m.def("cuda_mean_fwd", [](uptr A, uptr o, int nd, int dim, arr_i da) { ck(seera_cuda_mean_fwd(P<const F>(A), P<F>(o), nd, dim, da.data())); });
    m.def("cuda_max_fwd", [](uptr A, uptr o, int nd, int dim, arr_i da) { ck(seera_cuda_max_fwd(P<const F>(A), P<F>(o), nd, dim, da.data())); });
    m.def("cuda_min_fwd", [](uptr A, uptr o, int nd, int dim, arr_i da) { ck(seera_cuda_min_fwd(P<const F>(A), P<F>(o), nd, dim, da.data())); });
    m.def("cuda_argmax_fwd", [](uptr A, uptr o, int nd, int dim, arr_i da) { ck(seera_cuda_argmax_fwd(P<const F>(A), P<int>(o), nd, dim, da.data())); });
    m.def("cuda_argmin_fwd", [](uptr A, uptr o, int nd, int dim, arr_i da) { ck(seera_cuda_argmin_fwd(P<const F>(A), P<int>(o), nd, dim, da.data())); });
    m.def("cuda_sum_bwd", [](uptr d, uptr dA, int nd, int dim, arr_i da) { ck(seera_cuda_sum_bwd(P<const F>(d), P<F>(dA), nd, dim, da.data())); });
    m.def("cuda_mean_bwd", [](uptr d, uptr dA, int nd, int dim, arr_i da) { ck(seera_cuda_mean_bwd(P<const F>(d), P<F>(dA), nd, dim, da.data())); });
    m.def("cuda_max_bwd", [](uptr d, uptr fi, uptr fo, uptr dA, int nd, int dim, arr_i da) {
        ck(seera_cuda_max_bwd(P<const F>(d), P<const F>(fi), P<const F>(fo), P<F>(dA), nd, dim, da.data())); });
    m.def("cuda_min_bwd", [](uptr d, uptr fi, uptr fo, uptr dA, int nd, int dim, arr_i da) {
        ck(seera_cuda_min_bwd(P<const F>(d), P<const F>(fi), P<const F>(fo), P<F>(dA), nd, dim, da.data())); });

    // ---- scalar ops, fills, flat binary ops, broadcast ----------------------------------------------
    m.def("cuda_scaler_multiply_f", [](uptr a, float k, int n) { ck(seera_cuda_scaler_multiply_f(P<F>(a), k, n)); });
    m.def("cuda_scaler_add_f", [](uptr a, float k, int n) { ck(seera_cuda_scaler_add_f(P<F>(a), k, n)); });
    m.def("cuda_power_of", [](uptr a, float k, int n) { ck(seera_cuda_scaler_power_f(P<F>(a), k, n)); });
    m.def("cuda_ones_f", [](int n) { uptr p = ckp(seera_cuda_malloc_f32(n)); ck(seera_cuda_ones_f(P<F>(p), n)); return p; });
    m.def("cuda_zeros_f", [](int n) { uptr p = ckp(seera_cuda_malloc_f32(n)); ck(seera_cuda_zeros_f(P<F>(p), n)); return p; });
    m.def("cuda_elemadd", [](uptr A, uptr B, uptr C, int n) { ck(seera_cuda_elemadd_gputogpu(P<const F>(A), P<const F>(B), P<F>(C), n)); });
    m.def("cuda_elemsub", [](uptr A, uptr B, uptr C, int n) { ck(seera_cuda_elemsub_gputogpu(P<const F>(A), P<const F>(B), P<F>(C), n)); });
    m.def("cuda_elemdiv", [](uptr A, uptr B, uptr C, int n) { ck(seera_cuda_elemdiv_gputogpu(P<const F>(A), P<const F>(B), P<F>(C), n)); });
    m.def("cuda_elemmult", [](uptr A, uptr B, uptr C, int n) { ck(seera_cuda_elemmult_gputogpu(P<const F>(A), P<const F>(B), P<F>(C), n)); });
    m.def("broadcast_add_4d", [](uptr A, uptr B, uptr C, int aN, int aC, int aH, int aW, int bN, int bC, int bH, int bW) {
        ck(seera_broadcast_add_4d(P<const F>(A), P<const F>(B), P<F>(C), aN, aC, aH, aW, bN, bC, bH, bW)); });
    m.def("broadcast_mul_4d", [](uptr A, uptr B, uptr C, int aN, int aC, int aH, int aW, int bN, int bC, int bH, int bW) {
        ck(seera_broadcast_mul_4d(P<const F>(A), P<const F>(B), P<F>(C), aN, aC, aH, aW, bN, bC, bH, bW)); });

    // ---- additive entries (no counterpart in the reference binding) ---------------------------------
    m.def("init", [](int dev) { ck(seera_init(dev)); });
    m.def("stream_synchronize", []() { ck(seera_synchronize()); });
    m.def("set_stream", [](uptr s) { ck(seera_set_stream(P<void>(s))); });
    m.def("get_stream", []() { return reinterpret_cast<uptr>(seera_get_stream()); });
    m.def("last_status", []() { return seera_last_status(); });
    m.def("last_error", []() { return std::string(seera_last_error()); });
    m.def("clear_status", []() { seera_clear_status(); });
    m.def("launch_count", []() { return seera_launch_count(); });
    m.def("event_create", []() { return ckp(seera_event_create()); });
    m.def("event_record", [](uptr e) { ck(seera_event_record(P<void>(e))); });
    m.def("event_elapsed_ms", [](uptr a, uptr b) { return seera_event_elapsed_ms(P<void>(a), P<void>(b)); });
    m.def("event_destroy", [](uptr e) { ck(seera_event_destroy(P<void>(e))); });
    m.def("profile_enable", [](int on) { ck(seera_profile_enable(on)); });
    m.def("profile_read_kinds", []() {
        uint64_t n[3]; double ms[3], fl[3];
        ck(seera_profile_read_kinds(n, ms, fl));
        py::list out;
        for (int k = 0; k < 3; k++) out.append(py::make_tuple(n[k], ms[k], fl[k]));
        return out; });
    m.def("profile_report", []() {
        std::string buf(1 << 16, '\0');
        ck(seera_profile_report(&buf[0], buf.size()));
        py::list rows;
        size_t pos = 0, end = buf.find('\0');
        std::string text = buf.substr(0, end);
        while (pos < text.size()) {
            size_t nl = text.find('\n', pos);
            if (nl == std::string::npos) break;
            std::string line = text.substr(pos, nl - pos);
            pos = nl + 1;
            size_t t1 = line.find('\t'), t2 = line.find('\t', t1 + 1), t3 = line.find('\t', t2 + 1), t4 = line.find('\t', t3 + 1);
            rows.append(py::make_tuple(line.substr(0, t1), std::stoi(line.substr(t1 + 1, t2 - t1 - 1)),
                                       std::stoull(line.substr(t2 + 1, t3 - t2 - 1)), std::stod(line.substr(t3 + 1, t4 - t3 - 1)),
                                       std::stod(line.substr(t4 + 1))));
        }
        return rows; });
    m.def("profile_read", []() { uint64_t n = 0; double ms = 0, fl = 0; ck(seera_profile_read(&n, &ms, &fl)); return py::make_tuple(n, ms, fl); });
    m.def("set_precision", [](int mode) { ck(seera_set_precision(mode)); });
    m.def("graph_begin", []() { ck(seera_graph_begin()); });
    m.def("graph_end", []() { return ckp(seera_graph_end()); });
    m.def("graph_launch", [](uptr g) { ck(seera_graph_launch(P<void>(g))); });
    m.def("graph_destroy", [](uptr g) { ck(seera_graph_destroy(P<void>(g))); });
    m.def("is_capturing", []() { return seera_is_capturing() != 0; });
    m.def("cuda_adam_step_dev", [](uptr w, uptr g, uptr mm, uptr v, int n, uptr h) {
        ck(seera_adam_step_dev(P<F>(w), P<const F>(g), P<F>(mm), P<F>(v), n, P<const F>(h))); });
    m.def("cuda_sgd_step_dev", [](uptr w, uptr g, uptr vel, int n, uptr h) {
        ck(seera_sgd_step_dev(P<F>(w), P<const F>(g), P<F>(vel), n, P<const F>(h))); });
    m.def("set_option", [](const std::string &name, int v) { ck(seera_set_option(name.c_str(), v)); });
    m.def("tc_device_status", []() { return seera_tc_device_status(); });
    m.def("get_precision", []() { return seera_get_precision(); });
    m.def("pool_trim", []() { ck(seera_pool_trim()); });
    m.def("pool_bytes_reserved", []() { return seera_pool_bytes_reserved(); });
    m.def("upload_f32", [](uptr dst, arr_f a) { ck(seera_upload(P<void>(dst), a.data(), (size_t)a.size() * 4)); });
    m.def("upload_from_host_ptr", [](uptr dst, uptr host, size_t nbytes) { ck(seera_upload(P<void>(dst), P<const void>(host), nbytes)); });
    m.def("batchnorm_fwd", [](uptr x, uptr g, uptr b, uptr rm, uptr rv, uptr y, uptr mean, uptr si, int N, int C, int S, float momentum,
                              float eps, bool training) {
        ck(seera_batchnorm_fwd(P<const F>(x), P<const F>(g), P<const F>(b), P<F>(rm), P<F>(rv), P<F>(y), P<F>(mean), P<F>(si), N, C, S,
                               momentum, eps, training ? 1 : 0)); });
    m.def("batchnorm_bwd", [](uptr dy, uptr x, uptr mean, uptr si, uptr g, uptr dx, uptr dg, uptr db, int N, int C, int S) {
        ck(seera_batchnorm_bwd(P<const F>(dy), P<const F>(x), P<const F>(mean), P<const F>(si), P<const F>(g), P<F>(dx), P<F>(dg),
                               P<F>(db), N, C, S)); });
    m.def("batchnorm_fwd_sync", [](uptr x, uptr g, uptr b, uptr rm, uptr rv, uptr y, uptr mean, uptr si, int N, int C, int S, float momentum,
                              float eps, bool training) {
        ck(seera_batchnorm_fwd_sync(P<const F>(x), P<const F>(g), P<const F>(b), P<F>(rm), P<F>(rv), P<F>(y), P<F>(mean), P<F>(si), N, C, S,
                               momentum, eps, training ? 1 : 0)); });
    m.def("batchnorm_bwd_sync", [](uptr dy, uptr x, uptr mean, uptr si, uptr g, uptr dx, uptr dg, uptr db, int N, int C, int S) {
        ck(seera_batchnorm_bwd_sync(P<const F>(dy), P<const F>(x), P<const F>(mean), P<const F>(si), P<const F>(g), P<F>(dx), P<F>(dg),
                               P<F>(db), N, C, S)); });
    m.def("concat_fwd", [](uptr a, uptr b, uptr out, int N, int n1, int n2) { ck(seera_concat_fwd(P<const F>(a), P<const F>(b), P<F>(out), N, n1, n2)); });
    m.def("concat_bwd", [](uptr dout, uptr da, uptr db, int N, int n1, int n2) { ck(seera_concat_bwd(P<const F>(dout), P<F>(da), P<F>(db), N, n1, n2)); });
    m.def("onehot_f32", [](uptr labels, uptr out, int n, int classes) { ck(seera_onehot_f32(P<const int>(labels), P<F>(out), n, classes)); });
    m.def("stream_delay", [](int us) { ck(seera_stream_delay(us)); });
    m.def("copy_upload", [](uptr dst, uptr host, size_t nbytes) { ck(seera_copy_upload(P<void>(dst), P<const void>(host), nbytes)); });
    m.def("copy_download", [](uptr host, uptr src, size_t nbytes) { ck(seera_copy_download(P<void>(host), P<const void>(src), nbytes)); });
    m.def("copy_wait_compute", []() { ck(seera_copy_wait_compute()); });
    m.def("compute_wait_copy", []() { ck(seera_compute_wait_copy()); });
    m.def("copy_synchronize", []() { ck(seera_copy_synchronize()); });
    m.def("host_view", [](uptr p, size_t nbytes) {
        // NumPy view (uint8) of page-locked memory from host_alloc_pinned; the caller keeps the allocation alive
        return py::array_t<unsigned char>({nbytes}, {sizeof(unsigned char)}, P<unsigned char>(p), py::none()); });
    m.def("host_alloc_pinned", [](size_t n) { return ckp(seera_host_alloc_pinned(n)); });
    m.def("host_free_pinned", [](uptr p) { ck(seera_host_free_pinned(P<void>(p))); });
    m.def("bias_act_fwd", [](uptr z, uptr b, uptr y, int n, int ch, int inner, int act) {
        ck(seera_bias_act_fwd(P<const F>(z), P<const F>(b), P<F>(y), n, ch, inner, act)); });
    m.def("matmul_bias_act_fwd", [](uptr A, uptr B, uptr b, uptr C, int M, int N, int K, int act) {
        ck(seera_matmul_bias_act_fwd(P<const F>(A), P<const F>(B), P<const F>(b), P<F>(C), M, N, K, act)); });
    m.def("conv2d_bias_act_fwd", [](uptr x, uptr w, uptr b, uptr o, int N, int C, int H, int W, int Fo, int R, int S, int ph, int pw,
                                    int sh, int sw, int act) {
        ck(seera_conv2d_bias_act_fwd(P<const F>(x), P<const F>(w), P<const F>(b), P<F>(o), N, C, H, W, Fo, R, S, ph, pw, sh, sw, act)); });
    m.def("conv2DTranspose_bias_act_fwd", [](uptr x, uptr w, uptr b, uptr o, int N, int Ci, int H, int W, int Co, int KH, int KW,
                                             int sh, int sw, int ph, int pw, int act) {
        ck(seera_conv2DTranspose_bias_act_fwd(P<const F>(x), P<const F>(w), P<const F>(b), P<F>(o), N, Ci, H, W, Co, KH, KW, sh, sw, ph,
                                              pw, act)); });
    m.def("conv2d_bias_act_fwd_s", [](uptr x, uptr w, uptr b, uptr o, int N, int C, int H, int W, int Fo, int R, int S, int ph, int pw,
                                      int sh, int sw, int act, uptr x_in) {
        seera_shadow_t *keep = nullptr;
        ck(seera_conv2d_bias_act_fwd_s(P<const F>(x), P<const F>(w), P<const F>(b), P<F>(o), N, C, H, W, Fo, R, S, ph, pw, sh, sw, act,
                                       P<seera_shadow_t>(x_in), &keep));
        return reinterpret_cast<uptr>(keep); });
    m.def("maxpool2x2_fwd_s", [](uptr x, uptr o, uptr mask, int N, int C, int H, int W) {
        seera_shadow_t *keep = nullptr;
        ck(seera_maxpool2x2_fwd_s(P<const F>(x), P<F>(o), P<int>(mask), N, C, H, W, &keep));
        return reinterpret_cast<uptr>(keep); });
    m.def("conv2d_pool_fusable", [](int N, int C, int H, int W, int Fo, int R, int S, int sh, int sw, int ph, int pw) {
        return seera_conv2d_pool_fusable(N, C, H, W, Fo, R, S, sh, sw, ph, pw) != 0; });
    m.def("conv2d_bias_act_pool_fwd_s", [](uptr x, uptr w, uptr b, uptr pooled, uptr mask, int N, int C, int H, int W, int Fo, int R, int S,
                                           int ph, int pw, int sh, int sw, int act, uptr x_in, bool want_copies) {
        seera_shadow_t *keep = nullptr, *pc = nullptr;
        ck(seera_conv2d_bias_act_pool_fwd_s(P<const F>(x), P<const F>(w), P<const F>(b), P<F>(pooled), P<int>(mask), N, C, H, W, Fo, R, S,
                                            ph, pw, sh, sw, act, P<seera_shadow_t>(x_in), &keep, want_copies ? &pc : nullptr));
        return std::make_pair(reinterpret_cast<uptr>(keep), reinterpret_cast<uptr>(pc)); });
    m.def("shadow_free", [](uptr h) { seera_shadow_free(P<seera_shadow_t>(h)); });
    m.def("rows_free", [](uptr h) { seera_rows_free(P<seera_rows_t>(h)); });
    // Dense forward that keeps / hands on its operand copies: returns (a_keep, w_keep, c_copies) handles (0: none)
    m.def("matmul_bias_act_fwd_s", [](uptr a, uptr b, uptr bias, uptr c, int M, int N, int K, int act, uptr a_in, bool want_c_copies) {
        seera_rows_t *ak = nullptr, *wk = nullptr, *cc = nullptr;
        ck(seera_matmul_bias_act_fwd_s(P<const F>(a), P<const F>(b), P<const F>(bias), P<F>(c), M, N, K, act, P<seera_rows_t>(a_in), &ak, &wk,
                                       want_c_copies ? &cc : nullptr));
        return py::make_tuple(reinterpret_cast<uptr>(ak), reinterpret_cast<uptr>(wk), reinterpret_cast<uptr>(cc)); });
    m.def("matmul_act_bwd", [](uptr a, uptr b, uptr y, uptr g, uptr da, uptr db, uptr dbias, int M, int N, int K, int act, uptr a_keep,
                               uptr w_keep) {
        ck(seera_matmul_act_bwd(P<const F>(a), P<const F>(b), P<const F>(y), P<const F>(g), P<F>(da), P<F>(db), P<F>(dbias), M, N, K, act,
                                P<seera_rows_t>(a_keep), P<seera_rows_t>(w_keep))); });
    m.def("conv2d_act_bwd", [](uptr w, uptr x, uptr y, uptr g, uptr gp, uptr mask, uptr yp, uptr dx, uptr dw, uptr db, int N, int C, int H,
                               int W, int Fo, int R, int S, int sh, int sw, int ph, int pw, int act, uptr x_shadow) {
        ck(seera_conv2d_act_bwd(P<const F>(w), P<const F>(x), P<const F>(y), P<const F>(g), P<const F>(gp), P<const int>(mask),
                                P<const F>(yp), P<F>(dx),
                                P<F>(dw), P<F>(db), N, C, H, W, Fo, R, S, sh, sw, ph, pw, act, P<seera_shadow_t>(x_shadow))); });
    m.def("act_bias_bwd", [](uptr dy, uptr y, uptr dz, uptr db, int n, int ch, int inner, int act) {
        ck(seera_act_bias_bwd(P<const F>(dy), P<const F>(y), P<F>(dz), P<F>(db), n, ch, inner, act)); });
    m.def("softmax_cce_fwd_bwd", [](uptr z, uptr y, uptr p, uptr rows, uptr loss, uptr dz, int N, int C, float eps, float inv) {
        ck(seera_softmax_cce_fwd_bwd(P<const F>(z), P<const F>(y), P<F>(p), P<F>(rows), P<F>(loss), P<F>(dz), N, C, eps, inv)); });
    m.def("mse_partials", [](int n) { return seera_mse_partials(n); });
    m.def("mse_fwd_bwd", [](uptr p, uptr y, uptr part, uptr loss, uptr dp, int n, float inv) {
        ck(seera_mse_fwd_bwd(P<const F>(p), P<const F>(y), P<F>(part), P<F>(loss), P<F>(dp), n, inv)); });
    m.def("grad_scale_update", [](uptr g, long long n) { ck(seera_grad_scale_update(P<const F>(g), n)); });
    m.def("mae_fwd_bwd", [](uptr p, uptr y, uptr part, uptr loss, uptr dp, int n, float inv) {
        ck(seera_mae_fwd_bwd(P<const F>(p), P<const F>(y), P<F>(part), P<F>(loss), P<F>(dp), n, inv)); });
    m.def("bce_fwd_bwd", [](uptr p, uptr y, uptr part, uptr loss, uptr dp, int n, float inv, float eps) {
        ck(seera_bce_fwd_bwd(P<const F>(p), P<const F>(y), P<F>(part), P<F>(loss), P<F>(dp), n, inv, eps)); });
    m.def("cuda_adam_step", [](uptr w, uptr g, uptr mm, uptr v, int n, float lr, float b1, float omb1, float b2, float omb2,
                               float eps, float c1, float c2, float gs) {
        ck(seera_adam_step(P<F>(w), P<const F>(g), P<F>(mm), P<F>(v), n, lr, b1, omb1, b2, omb2, eps, c1, c2, gs)); });
    m.def("cuda_sgd_step", [](uptr w, uptr g, uptr vel, int n, float lr, float mu, float gs) {
        ck(seera_sgd_step(P<F>(w), P<const F>(g), P<F>(vel), n, lr, mu, gs)); });

    // ---- data parallel (NCCL inside the engine) ----
    m.def("dp_unique_id", []() {
        std::string id((size_t)seera_dp_unique_id_bytes(), '\0');
        ck(seera_dp_unique_id(&id[0], (int)id.size()));
        return py::bytes(id); });
    m.def("dp_init", [](int rank, int world, py::bytes id) {
        std::string s = id;
        py::gil_scoped_release nogil;           // collective over the ranks: may wait for the others
        ck(seera_dp_init(rank, world, s.data(), (int)s.size())); });
    m.def("dp_rank", []() { return seera_dp_rank(); });
    m.def("dp_world", []() { return seera_dp_world(); });
    m.def("dp_nccl_version", []() { return seera_dp_nccl_version(); });
    m.def("dp_alloc", [](size_t bytes) { return ckp(seera_dp_alloc(bytes)); });
    m.def("dp_free", [](uptr p) { ck(seera_dp_free(P<void>(p))); });
    m.def("dp_allreduce", [](uptr p, long long n, int op) { ck(seera_dp_allreduce(P<F>(p), n, op)); });
    m.def("dp_broadcast", [](uptr p, long long n, int root) { ck(seera_dp_broadcast(P<F>(p), n, root)); });
    m.def("dp_reduce_range", [](uptr p, long long b, long long e) { ck(seera_dp_reduce_range(P<F>(p), b, e)); });
    m.def("dp_join", []() { ck(seera_dp_join()); });
    m.def("dp_side_begin", []() { ck(seera_dp_side_begin()); });
    m.def("dp_side_end", []() { ck(seera_dp_side_end()); });
    m.def("dp_poll", []() { ck(seera_dp_poll()); });
    m.def("dp_wait_host", [](int timeout_ms) { py::gil_scoped_release nogil; ck(seera_dp_wait_host(timeout_ms)); });
    m.def("dp_abort", []() { ck(seera_dp_abort()); });
    m.def("dp_finalize", []() { ck(seera_dp_finalize()); });
}
