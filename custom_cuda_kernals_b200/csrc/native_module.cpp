// `_native`: the Python-facing validation + FFI layer over the C ABI in
// include/custom_cuda_b200.h.
//
// C++ stand-in for the reference's Rust/PyO3 module (src/lib.rs:11-29 and
// src/kernels/*.rs): the same function names and argument orders, the same
// checks in the same spirit (device type, contiguity, dtype set, dtype and
// shape relations -> ValueError; a non-zero cudaError_t from a launcher ->
// RuntimeError), the same zero-copy contract (raw data_ptr() of caller-owned
// tensors, launch on torch's current stream of the first tensor's device, no
// allocation or synchronisation).  Two additions the reference lacks: every
// tensor of a call must live on the same device, and the device is made
// current for the duration of the call.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <sstream>
#include <tuple>
#include <string>
#include <vector>

#include "../../include/custom_cuda_b200.h"

namespace {

namespace py = pybind11;

std::string shape_str(const at::Tensor& t) {
    std::ostringstream os;
    os << "[";
    for (int64_t i = 0; i < t.dim(); ++i) os << (i ? ", " : "") << t.size(i);
    os << "]";
    return os.str();
}

const char* tag_name(int32_t tag) {
    switch (tag) {
        case CCK_F32: return "F32";
        case CCK_F16: return "F16";
        case CCK_BF16: return "BF16";
        case CCK_F8E4M3: return "F8E4M3";
        case CCK_F8E5M2: return "F8E5M2";
        default: return "?";
    }
}

[[noreturn]] void value_error(const std::string& msg) { throw py::value_error(msg); }

// device type + contiguity (src/kernels/tensor.rs:38-62)
void check_cuda_contiguous(const char* name, const at::Tensor& t) {
    if (!t.is_cuda())
        value_error(std::string("argument '") + name + "' must be a CUDA tensor, got device type '" +
                    c10::DeviceTypeName(t.device().type(), /*lower_case=*/true) + "'");
    if (!t.is_contiguous()) value_error(std::string("argument '") + name + "' must be contiguous");
}

// compute / storage dtype tag (src/kernels/dtype.rs:14-25)
int32_t tag_of(const char* name, const at::Tensor& t) {
    check_cuda_contiguous(name, t);
    switch (t.scalar_type()) {
        case at::kFloat: return CCK_F32;
        case at::kHalf: return CCK_F16;
        case at::kBFloat16: return CCK_BF16;
        case at::kFloat8_e4m3fn: return CCK_F8E4M3;
        case at::kFloat8_e5m2: return CCK_F8E5M2;
        default:
            value_error(std::string("unsupported dtype '") + c10::toString(t.scalar_type()) +
                        "'; expected float32, float16, or bfloat16");
    }
}

void expect_float_input(const char* name, int32_t tag) {
    if (tag != CCK_F32 && tag != CCK_F16 && tag != CCK_BF16)
        value_error(std::string("unsupported dtype '") + tag_name(tag) + "' for '" + name +
                    "'; expected float32, float16, or bfloat16");
}

void expect_same_dtype(const char* name, int32_t got, int32_t want) {
    if (got != want)
        value_error(std::string("dtype mismatch: '") + name + "' is " + tag_name(got) + " but expected " +
                    tag_name(want) + " (must match 'x')");
}

void expect_f32(const char* name, int32_t tag, const char* why = "") {
    if (tag != CCK_F32)
        value_error(std::string("unsupported dtype '") + name + " must be float32" + why + ", got " + tag_name(tag) + "'");
}

void expect_int(const char* name, const at::Tensor& t, at::ScalarType want, const char* want_name) {
    check_cuda_contiguous(name, t);
    if (t.scalar_type() != want)
        value_error(std::string("unsupported dtype '") + name + " must be " + want_name + ", got " +
                    c10::toString(t.scalar_type()) + "'");
}

// All tensors of a call on one device; returns a guard-ready device index.
struct Launch {
    c10::cuda::CUDAGuard guard;
    void* stream;
    explicit Launch(const at::Tensor& first, std::initializer_list<const at::Tensor*> rest)
        : guard(first.device()), stream(nullptr) {
        for (const at::Tensor* t : rest)
            if (t->defined() && t->device() != first.device())
                value_error("all tensors must be on the same CUDA device; got " + first.device().str() + " and " +
                            t->device().str());
        stream = c10::cuda::getCurrentCUDAStream(first.device().index()).stream();
    }
};

void check_launch(const char* fn, int32_t err) {
    if (err != 0)
        throw std::runtime_error(std::string("CUDA error: ") + fn + " failed, cudaError_t = " + std::to_string(err));
}

int32_t parse_fp8_format(const std::string& s) {
    if (s == "e4m3") return CCK_F8E4M3;
    if (s == "e5m2") return CCK_F8E5M2;
    value_error("fp8_format must be 'e4m3' or 'e5m2', got '" + s + "'");
}

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ------------------------------------------------------------------ src/kernels/rmsnorm_residual.rs:46-115
void rmsnorm_residual_fwd(const at::Tensor& x, const at::Tensor& residual, const at::Tensor& weight,
                          const at::Tensor& y, const at::Tensor& residual_out, double eps) {
    const int32_t dt = tag_of("x", x);
    expect_float_input("x", dt);
    expect_same_dtype("residual", tag_of("residual", residual), dt);
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    expect_same_dtype("residual_out", tag_of("residual_out", residual_out), dt);
    if (residual.sizes() != x.sizes() || y.sizes() != x.sizes() || residual_out.sizes() != x.sizes())
        value_error("shape mismatch: x/residual/y/residual_out must share the same shape; got x=" + shape_str(x) +
                    ", residual=" + shape_str(residual) + ", y=" + shape_str(y) +
                    ", residual_out=" + shape_str(residual_out));
    if (x.dim() < 1) value_error("shape mismatch: x must have at least 1 dimension");
    const int64_t cols = x.size(-1);
    if (weight.dim() != 1 || weight.size(0) != cols)
        value_error("shape mismatch: weight shape " + shape_str(weight) + " must be [" + std::to_string(cols) +
                    "] (x's last dimension)");
    const int64_t rows = cols > 0 ? x.numel() / cols : 0;
    Launch l(x, {&residual, &weight, &y, &residual_out});
    check_launch("launch_rmsnorm_residual_fwd",
                 launch_rmsnorm_residual_fwd(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), y.data_ptr(),
                                             residual_out.data_ptr(), rows, cols, static_cast<float>(eps), dt,
                                             l.stream));
}

// the norm alone (no counterpart in the reference)
void rmsnorm_fwd(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& y, double eps) {
    const int32_t dt = tag_of("x", x);
    expect_float_input("x", dt);
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    if (y.sizes() != x.sizes())
        value_error("shape mismatch: x and y must share the same shape; got x=" + shape_str(x) + ", y=" + shape_str(y));
    if (x.dim() < 1) value_error("shape mismatch: x must have at least 1 dimension");
    const int64_t cols = x.size(-1);
    if (weight.dim() != 1 || weight.size(0) != cols)
        value_error("shape mismatch: weight shape " + shape_str(weight) + " must be [" + std::to_string(cols) +
                    "] (x's last dimension)");
    const int64_t rows = cols > 0 ? x.numel() / cols : 0;
    Launch l(x, {&weight, &y});
    check_launch("launch_rmsnorm_fwd", launch_rmsnorm_fwd(x.data_ptr(), weight.data_ptr(), y.data_ptr(), rows, cols,
                                                          static_cast<float>(eps), dt, l.stream));
}

// ------------------------------------------------------------------ src/kernels/swiglu.rs:31-79
void swiglu_fwd(const at::Tensor& gate, const at::Tensor& up, const at::Tensor& y) {
    const int32_t dt = tag_of("gate", gate);
    expect_float_input("gate", dt);
    expect_same_dtype("up", tag_of("up", up), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    if (up.sizes() != gate.sizes() || y.sizes() != gate.sizes())
        value_error("shape mismatch: gate/up/y must share the same shape; got gate=" + shape_str(gate) +
                    ", up=" + shape_str(up) + ", y=" + shape_str(y));
    Launch l(gate, {&up, &y});
    check_launch("launch_swiglu_fwd",
                 launch_swiglu_fwd(gate.data_ptr(), up.data_ptr(), y.data_ptr(), gate.numel(), dt, l.stream));
}

// ------------------------------------------------------------------ src/kernels/moe_router.rs, token_permute.rs
void moe_router_fwd(const at::Tensor& logits, const at::Tensor& topk_weights, const at::Tensor& topk_indices,
                    bool renormalize) {
    const int32_t dt = tag_of("logits", logits);
    expect_float_input("logits", dt);
    const int32_t wdt = tag_of("topk_weights", topk_weights);
    expect_int("topk_indices", topk_indices, at::kLong, "int64");
    if (wdt != CCK_F32)
        value_error(std::string("unsupported dtype 'topk_weights must be float32, got ") + tag_name(wdt) + "'");
    if (logits.dim() != 2)
        value_error("shape mismatch: logits must be 2-D [num_tokens, num_experts], got " + shape_str(logits));
    const int64_t t = logits.size(0), e = logits.size(1);
    if (topk_weights.dim() != 2 || topk_weights.size(0) != t)
        value_error("shape mismatch: topk_weights shape " + shape_str(topk_weights) + " must be [" + std::to_string(t) + ", k]");
    const int64_t k = topk_weights.size(1);
    if (topk_indices.dim() != 2 || topk_indices.size(0) != t || topk_indices.size(1) != k)
        value_error("shape mismatch: topk_indices shape " + shape_str(topk_indices) + " must match topk_weights' [" +
                    std::to_string(t) + ", " + std::to_string(k) + "]");
    if (k > e) throw std::runtime_error("k (" + std::to_string(k) + ") must be <= num_experts (" + std::to_string(e) + ")");
    if (e > 256)
        value_error("shape mismatch: num_experts (" + std::to_string(e) + ") exceeds this kernel's supported maximum of 256");
    if (t == 0 || k == 0) return;
    Launch l(logits, {&topk_weights, &topk_indices});
    check_launch("launch_moe_router_fwd",
                 launch_moe_router_fwd(logits.data_ptr(), static_cast<float*>(topk_weights.data_ptr()),
                                       static_cast<int64_t*>(topk_indices.data_ptr()), t, e, k, dt, renormalize ? 1 : 0,
                                       l.stream));
}

void token_gather_fwd(const at::Tensor& src, const at::Tensor& indices, const at::Tensor& dst) {
    const int32_t dt = tag_of("src", src);
    expect_float_input("src", dt);
    expect_int("indices", indices, at::kLong, "int64");
    expect_same_dtype("dst", tag_of("dst", dst), dt);
    if (src.dim() != 2 || dst.dim() != 2)
        value_error("shape mismatch: src and dst must be 2-D; got src=" + shape_str(src) + ", dst=" + shape_str(dst));
    const int64_t h = src.size(1);
    if (dst.size(1) != h)
        value_error("shape mismatch: dst's hidden dim (" + std::to_string(dst.size(1)) + ") must match src's (" +
                    std::to_string(h) + ")");
    if (indices.dim() != 1 || indices.size(0) != dst.size(0))
        value_error("shape mismatch: indices shape " + shape_str(indices) + " must be [" + std::to_string(dst.size(0)) +
                    "] (dst's row count)");
    Launch l(src, {&indices, &dst});
    check_launch("launch_token_gather_fwd",
                 launch_token_gather_fwd(src.data_ptr(), static_cast<const int64_t*>(indices.data_ptr()), dst.data_ptr(),
                                         dst.size(0), h, dt, l.stream));
}

void token_combine_fwd(const at::Tensor& expert_output, const at::Tensor& unpermute_index, const at::Tensor& weights,
                       const at::Tensor& combined) {
    const int32_t dt = tag_of("expert_output", expert_output);
    expect_float_input("expert_output", dt);
    expect_int("unpermute_index", unpermute_index, at::kLong, "int64");
    const int32_t wdt = tag_of("weights", weights);
    expect_same_dtype("combined", tag_of("combined", combined), dt);
    if (wdt != CCK_F32) value_error(std::string("unsupported dtype 'weights must be float32, got ") + tag_name(wdt) + "'");
    if (expert_output.dim() != 2 || combined.dim() != 2)
        value_error("shape mismatch: expert_output and combined must be 2-D; got expert_output=" +
                    shape_str(expert_output) + ", combined=" + shape_str(combined));
    const int64_t h = expert_output.size(1);
    if (combined.size(1) != h)
        value_error("shape mismatch: combined's hidden dim (" + std::to_string(combined.size(1)) +
                    ") must match expert_output's (" + std::to_string(h) + ")");
    if (unpermute_index.dim() != 2 || weights.dim() != 2)
        value_error("shape mismatch: unpermute_index and weights must be 2-D [T, k]; got unpermute_index=" +
                    shape_str(unpermute_index) + ", weights=" + shape_str(weights));
    const int64_t t = unpermute_index.size(0), k = unpermute_index.size(1);
    if (weights.size(0) != t || weights.size(1) != k)
        value_error("shape mismatch: weights shape " + shape_str(weights) + " must match unpermute_index's [" +
                    std::to_string(t) + ", " + std::to_string(k) + "]");
    if (combined.size(0) != t)
        value_error("shape mismatch: combined's row count (" + std::to_string(combined.size(0)) +
                    ") must match unpermute_index's [" + std::to_string(t) + ", ...]");
    Launch l(expert_output, {&unpermute_index, &weights, &combined});
    check_launch("launch_token_combine_fwd",
                 launch_token_combine_fwd(expert_output.data_ptr(), static_cast<const int64_t*>(unpermute_index.data_ptr()),
                                          static_cast<const float*>(weights.data_ptr()), combined.data_ptr(), t, k, h, dt,
                                          l.stream));
}

// expert-parallel row exchange (no counterpart in the reference)
void token_dispatch_fwd(const at::Tensor& src, const at::Tensor& src_row, const at::Tensor& dst_rank,
                        const at::Tensor& dst_row, const at::Tensor& dst_bases, int64_t capacity_rows) {
    const int32_t dt = tag_of("src", src);
    expect_float_input("src", dt);
    expect_int("src_row", src_row, at::kLong, "int64");
    expect_int("dst_rank", dst_rank, at::kLong, "int64");
    expect_int("dst_row", dst_row, at::kLong, "int64");
    expect_int("dst_bases", dst_bases, at::kLong, "int64");
    if (src.dim() != 2) value_error("shape mismatch: src must be 2-D [rows, hidden], got " + shape_str(src));
    const int64_t n = src_row.numel();
    if (dst_rank.numel() != n || dst_row.numel() != n)
        value_error("shape mismatch: src_row, dst_rank and dst_row must have the same number of elements");
    if (dst_bases.dim() != 1 || dst_bases.numel() < 1) value_error("shape mismatch: dst_bases must be a 1-D table of addresses");
    if ((src.size(1) * src.element_size()) % 16 != 0) value_error("shape mismatch: a row must be a multiple of 16 bytes");
    if (capacity_rows < 0) value_error("capacity_rows must not be negative");
    Launch l(src, {&src_row, &dst_rank, &dst_row, &dst_bases});
    check_launch("launch_token_dispatch_fwd",
                 launch_token_dispatch_fwd(src.data_ptr(), static_cast<const int64_t*>(src_row.data_ptr()),
                                           static_cast<const int64_t*>(dst_rank.data_ptr()),
                                           static_cast<const int64_t*>(dst_row.data_ptr()),
                                           static_cast<const int64_t*>(dst_bases.data_ptr()), dst_bases.numel(),
                                           capacity_rows, src.size(0), n, src.size(1), dt, l.stream));
}

void ep_plan(const at::Tensor& topk, const at::Tensor& counts, int64_t rank, const at::Tensor& src_row,
             const at::Tensor& dst_rank, const at::Tensor& dst_row, const at::Tensor& pull_rank,
             const at::Tensor& pull_row, const at::Tensor& meta) {
    expect_int("topk", topk, at::kLong, "int64");
    expect_int("counts", counts, at::kLong, "int64");
    for (const auto& named : {std::make_pair("src_row", &src_row), std::make_pair("dst_rank", &dst_rank),
                              std::make_pair("dst_row", &dst_row), std::make_pair("pull_rank", &pull_rank),
                              std::make_pair("pull_row", &pull_row), std::make_pair("meta", &meta)})
        expect_int(named.first, *named.second, at::kLong, "int64");
    if (topk.dim() != 2 || counts.dim() != 2) value_error("shape mismatch: topk must be [T, k] and counts [world, experts]");
    const int64_t n = topk.numel(), k = topk.size(1), world = counts.size(0), experts = counts.size(1);
    if (src_row.numel() != n || dst_rank.numel() != n || dst_row.numel() != n || pull_rank.numel() != n ||
        pull_row.numel() != n || meta.numel() != 2)
        value_error("shape mismatch: the five route outputs need T * k elements each, meta 2");
    if (experts > 256 || world > 32 || world < 1 || experts % world != 0 || k < 1)
        value_error("shape mismatch: at most 256 experts and 32 ranks, experts divisible by the ranks");
    if (rank < 0 || rank >= world) value_error("rank must lie in [0, world)");
    Launch l(topk, {&counts, &src_row, &dst_rank, &dst_row, &pull_rank, &pull_row, &meta});
    check_launch("launch_ep_plan",
                 launch_ep_plan(static_cast<const int64_t*>(topk.data_ptr()), static_cast<const int64_t*>(counts.data_ptr()),
                                n, k, world, experts, rank, static_cast<int64_t*>(src_row.data_ptr()),
                                static_cast<int64_t*>(dst_rank.data_ptr()), static_cast<int64_t*>(dst_row.data_ptr()),
                                static_cast<int64_t*>(pull_rank.data_ptr()), static_cast<int64_t*>(pull_row.data_ptr()),
                                static_cast<int64_t*>(meta.data_ptr()), l.stream));
}

void token_combine_remote_fwd(const at::Tensor& src_bases, int64_t capacity_rows, const at::Tensor& src_rank,
                              const at::Tensor& src_row, const at::Tensor& weights, const at::Tensor& combined) {
    const int32_t dt = tag_of("combined", combined);
    expect_float_input("combined", dt);
    expect_int("src_bases", src_bases, at::kLong, "int64");
    expect_int("src_rank", src_rank, at::kLong, "int64");
    expect_int("src_row", src_row, at::kLong, "int64");
    expect_f32("weights", tag_of("weights", weights));
    if (combined.dim() != 2) value_error("shape mismatch: combined must be 2-D [T, hidden], got " + shape_str(combined));
    if (src_rank.dim() != 2 || src_rank.size(0) != combined.size(0) || src_row.sizes() != src_rank.sizes() ||
        weights.sizes() != src_rank.sizes())
        value_error("shape mismatch: src_rank, src_row and weights must be [T, k] with T = combined's rows; got " +
                    shape_str(src_rank) + ", " + shape_str(src_row) + ", " + shape_str(weights));
    const int64_t per_vec = dt == CCK_F32 ? 4 : 8;
    if (combined.size(1) % per_vec != 0) value_error("shape mismatch: hidden must be a multiple of " + std::to_string(per_vec));
    if (src_bases.dim() != 1 || src_bases.numel() < 1) value_error("shape mismatch: src_bases must be a 1-D table of addresses");
    Launch l(combined, {&src_bases, &src_rank, &src_row, &weights});
    check_launch("launch_token_combine_remote_fwd",
                 launch_token_combine_remote_fwd(static_cast<const int64_t*>(src_bases.data_ptr()), src_bases.numel(),
                                                 capacity_rows, static_cast<const int64_t*>(src_rank.data_ptr()),
                                                 static_cast<const int64_t*>(src_row.data_ptr()),
                                                 static_cast<const float*>(weights.data_ptr()), combined.data_ptr(),
                                                 combined.size(0), src_rank.size(1), combined.size(1), dt, l.stream));
}

// gradients of the two ops above (no counterpart in the reference)
void swiglu_bwd(const at::Tensor& gate, const at::Tensor& up, const at::Tensor& dy, const at::Tensor& dgate,
                const at::Tensor& dup) {
    const int32_t dt = tag_of("gate", gate);
    expect_float_input("gate", dt);
    expect_same_dtype("up", tag_of("up", up), dt);
    expect_same_dtype("dy", tag_of("dy", dy), dt);
    expect_same_dtype("dgate", tag_of("dgate", dgate), dt);
    expect_same_dtype("dup", tag_of("dup", dup), dt);
    if (up.sizes() != gate.sizes() || dy.sizes() != gate.sizes() || dgate.sizes() != gate.sizes() ||
        dup.sizes() != gate.sizes())
        value_error("shape mismatch: gate/up/dy/dgate/dup must share the same shape; got gate=" + shape_str(gate) +
                    ", up=" + shape_str(up) + ", dy=" + shape_str(dy));
    Launch l(gate, {&up, &dy, &dgate, &dup});
    check_launch("launch_swiglu_bwd", launch_swiglu_bwd(gate.data_ptr(), up.data_ptr(), dy.data_ptr(), dgate.data_ptr(),
                                                        dup.data_ptr(), gate.numel(), dt, l.stream));
}

void rmsnorm_residual_bwd(const at::Tensor& dy, const c10::optional<at::Tensor>& d_residual_out,
                          const at::Tensor& residual_out, const at::Tensor& weight, const at::Tensor& dx,
                          const at::Tensor& dweight, const at::Tensor& workspace, double eps) {
    const int32_t dt = tag_of("dy", dy);
    expect_float_input("dy", dt);
    expect_same_dtype("residual_out", tag_of("residual_out", residual_out), dt);
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("dx", tag_of("dx", dx), dt);
    expect_same_dtype("dweight", tag_of("dweight", dweight), dt);
    check_cuda_contiguous("workspace", workspace);
    if (residual_out.sizes() != dy.sizes() || dx.sizes() != dy.sizes())
        value_error("shape mismatch: dy/residual_out/dx must share the same shape; got dy=" + shape_str(dy) +
                    ", residual_out=" + shape_str(residual_out) + ", dx=" + shape_str(dx));
    if (dy.dim() < 1) value_error("shape mismatch: dy must have at least 1 dimension");
    const int64_t cols = dy.size(-1);
    if (weight.dim() != 1 || weight.size(0) != cols || dweight.dim() != 1 || dweight.size(0) != cols)
        value_error("shape mismatch: weight and dweight must be [" + std::to_string(cols) + "]");
    const void* dro = nullptr;
    if (d_residual_out.has_value()) {
        expect_same_dtype("d_residual_out", tag_of("d_residual_out", *d_residual_out), dt);
        if (d_residual_out->sizes() != dy.sizes())
            value_error("shape mismatch: d_residual_out shape " + shape_str(*d_residual_out) + " must match dy " + shape_str(dy));
        dro = d_residual_out->data_ptr();
    }
    const int64_t rows = cols > 0 ? dy.numel() / cols : 0;
    const int64_t per_vec = dt == CCK_F32 ? 4 : 8;
    if (cols % per_vec != 0 || cols / per_vec > 1024)
        value_error("shape mismatch: the gradient kernel needs a column count that is a multiple of " +
                    std::to_string(per_vec) + " and at most " + std::to_string(1024 * per_vec));
    const int64_t ws_bytes = static_cast<int64_t>(workspace.numel()) * workspace.element_size();
    if (ws_bytes < cck_rmsnorm_bwd_workspace_bytes(rows, cols))
        value_error("shape mismatch: workspace has " + std::to_string(ws_bytes) + " bytes, needs " +
                    std::to_string(cck_rmsnorm_bwd_workspace_bytes(rows, cols)));
    const at::Tensor undefined;
    Launch l(dy, {&residual_out, &weight, &dx, &dweight, &workspace,
                  d_residual_out.has_value() ? &*d_residual_out : &undefined});
    check_launch("launch_rmsnorm_residual_bwd",
                 launch_rmsnorm_residual_bwd(dy.data_ptr(), dro, residual_out.data_ptr(), weight.data_ptr(), dx.data_ptr(),
                                             dweight.data_ptr(), workspace.data_ptr(), ws_bytes, rows, cols,
                                             static_cast<float>(eps), dt, l.stream));
}

int64_t rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t cols) { return cck_rmsnorm_bwd_workspace_bytes(rows, cols); }

// ------------------------------------------------------------------ src/kernels/rope.rs:42-153
void rope_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& cos, const at::Tensor& sin,
              const at::Tensor& q_out, const at::Tensor& k_out) {
    const int32_t dt = tag_of("q", q);
    expect_float_input("q", dt);
    const int32_t kdt = tag_of("k", k);
    const int32_t cdt = tag_of("cos", cos), sdt = tag_of("sin", sin);
    expect_same_dtype("k", kdt, dt);
    expect_same_dtype("q_out", tag_of("q_out", q_out), dt);
    expect_same_dtype("k_out", tag_of("k_out", k_out), kdt);
    expect_f32("cos", cdt, " (RoPE tables are always fp32)");
    expect_f32("sin", sdt, " (RoPE tables are always fp32)");
    if (q.dim() != 4)
        value_error("shape mismatch: q must be 4-D [batch, seq_len, n_q_heads, head_dim], got " + shape_str(q));
    if (k.dim() != 4)
        value_error("shape mismatch: k must be 4-D [batch, seq_len, n_kv_heads, head_dim], got " + shape_str(k));
    if (q_out.sizes() != q.sizes()) value_error("shape mismatch: q_out must match q's shape");
    if (k_out.sizes() != k.sizes()) value_error("shape mismatch: k_out must match k's shape");
    const int64_t batch = q.size(0), seq = q.size(1), hq = q.size(2), d = q.size(3);
    if (k.size(0) != batch || k.size(1) != seq || k.size(3) != d)
        value_error("shape mismatch: q and k must share batch/seq_len/head_dim; got q=" + shape_str(q) +
                    ", k=" + shape_str(k));
    if (d % 2 != 0) value_error("shape mismatch: head_dim must be even, got " + std::to_string(d));
    const int64_t half = d / 2;
    if (cos.dim() != 2 || sin.dim() != 2 || cos.size(0) != seq || cos.size(1) != half || sin.size(0) != seq ||
        sin.size(1) != half)
        value_error("shape mismatch: cos/sin must have shape [" + std::to_string(seq) + ", " + std::to_string(half) +
                    "]; got cos=" + shape_str(cos) + ", sin=" + shape_str(sin));
    Launch l(q, {&k, &cos, &sin, &q_out, &k_out});
    check_launch("launch_rope_fwd",
                 launch_rope_fwd(q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), q_out.data_ptr(),
                                 k_out.data_ptr(), batch, seq, hq, k.size(2), d, dt, l.stream));
}

// rope on strided q/k views (no counterpart in the reference): q [B,S,Hq,D] and k [B,S,Hkv,D] may be
// views whose tokens are a fixed number of elements apart (heads of a token contiguous)
int64_t token_stride_of(const char* name, const at::Tensor& t) {
    if (!t.is_cuda())
        value_error(std::string("argument '") + name + "' must be a CUDA tensor, got device type '" +
                    c10::DeviceTypeName(t.device().type(), true) + "'");
    if (t.dim() != 4) value_error(std::string("shape mismatch: ") + name + " must be 4-D [batch, seq_len, heads, head_dim], got " + shape_str(t));
    const int64_t s = t.size(1), h = t.size(2), d = t.size(3);
    // a dimension of size 1 carries no usable stride: one position per sequence is spaced by the batch stride
    const int64_t ts = s > 1 ? t.stride(1) : (t.size(0) > 1 ? t.stride(0) : h * d);
    const bool ok = t.stride(3) == 1 && (h == 1 || t.stride(2) == d) &&
                    (t.size(0) == 1 || s == 1 || t.stride(0) == s * ts) && ts >= h * d;
    if (!ok) value_error(std::string("argument '") + name + "' must have contiguous heads per token and evenly spaced tokens");
    return ts;
}

void rope_strided_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& cos, const at::Tensor& sin,
                      const at::Tensor& q_out, const at::Tensor& k_out) {
    const int64_t qs = token_stride_of("q", q), ks = token_stride_of("k", k);
    int32_t dt;
    switch (q.scalar_type()) {
        case at::kFloat: dt = CCK_F32; break;
        case at::kHalf: dt = CCK_F16; break;
        case at::kBFloat16: dt = CCK_BF16; break;
        default: value_error(std::string("unsupported dtype '") + c10::toString(q.scalar_type()) + "'; expected float32, float16, or bfloat16");
    }
    if (k.scalar_type() != q.scalar_type()) value_error("dtype mismatch: 'k' must match 'q'");
    expect_same_dtype("q_out", tag_of("q_out", q_out), dt);
    expect_same_dtype("k_out", tag_of("k_out", k_out), dt);
    expect_f32("cos", tag_of("cos", cos), " (RoPE tables are always fp32)");
    expect_f32("sin", tag_of("sin", sin), " (RoPE tables are always fp32)");
    if (q_out.sizes() != q.sizes()) value_error("shape mismatch: q_out must match q's shape");
    if (k_out.sizes() != k.sizes()) value_error("shape mismatch: k_out must match k's shape");
    const int64_t batch = q.size(0), seq = q.size(1), hq = q.size(2), d = q.size(3);
    if (k.size(0) != batch || k.size(1) != seq || k.size(3) != d)
        value_error("shape mismatch: q and k must share batch/seq_len/head_dim; got q=" + shape_str(q) + ", k=" + shape_str(k));
    if (d % 2 != 0) value_error("shape mismatch: head_dim must be even, got " + std::to_string(d));
    if (cos.dim() != 2 || sin.dim() != 2 || cos.size(0) != seq || cos.size(1) != d / 2 || sin.size(0) != seq ||
        sin.size(1) != d / 2)
        value_error("shape mismatch: cos/sin must have shape [" + std::to_string(seq) + ", " + std::to_string(d / 2) + "]");
    Launch l(q, {&k, &cos, &sin, &q_out, &k_out});
    check_launch("launch_rope_strided_fwd",
                 launch_rope_strided_fwd(q.data_ptr(), k.data_ptr(), cos.data_ptr(), sin.data_ptr(), q_out.data_ptr(),
                                         k_out.data_ptr(), batch, seq, hq, k.size(2), d, qs, ks, dt, l.stream));
}

// ------------------------------------------------------------------ src/kernels/fp8_quant.rs:62-210 (+ token)
struct Fp8Args {
    int32_t dt, fmt;
    int64_t m, n;
};

Fp8Args fp8_common(const at::Tensor& x, const at::Tensor& x_fp8, const at::Tensor& scale, const std::string& format) {
    Fp8Args a;
    a.fmt = parse_fp8_format(format);
    a.dt = tag_of("x", x);
    expect_float_input("x", a.dt);
    const int32_t odt = tag_of("x_fp8", x_fp8);
    const int32_t sdt = tag_of("scale", scale);
    if (odt != a.fmt)
        value_error(std::string("unsupported dtype 'x_fp8 dtype ") + tag_name(odt) +
                    " does not match requested fp8_format \"" + format + "\"'");
    expect_f32("scale", sdt);
    if (x.dim() != 2) value_error("shape mismatch: x must be 2-D [M, N]; got " + shape_str(x));
    a.m = x.size(0);
    a.n = x.size(1);
    if (x_fp8.dim() != 2 || x_fp8.size(0) != a.m || x_fp8.size(1) != a.n)
        value_error("shape mismatch: x_fp8 shape " + shape_str(x_fp8) + " must be [" + std::to_string(a.m) + ", " +
                    std::to_string(a.n) + "]");
    return a;
}

void fp8_quant_block_fwd(const at::Tensor& x, const at::Tensor& x_fp8, const at::Tensor& scale,
                         const std::string& fp8_format) {
    const Fp8Args a = fp8_common(x, x_fp8, scale, fp8_format);
    const int64_t rb = ceil_div(a.m, 128), cb = ceil_div(a.n, 128);
    if (scale.dim() != 2 || scale.size(0) != rb || scale.size(1) != cb)
        value_error("shape mismatch: scale shape " + shape_str(scale) + " must be [" + std::to_string(rb) + ", " +
                    std::to_string(cb) + "] (ceil(M/128), ceil(N/128))");
    Launch l(x, {&x_fp8, &scale});
    check_launch("launch_fp8_quant_block_fwd",
                 launch_fp8_quant_block_fwd(x.data_ptr(), static_cast<uint8_t*>(x_fp8.data_ptr()),
                                            static_cast<float*>(scale.data_ptr()), a.m, a.n, a.dt, a.fmt, l.stream));
}

void fp8_quant_tensor_fwd(const at::Tensor& x, const at::Tensor& x_fp8, const at::Tensor& scale,
                          const at::Tensor& amax_scratch, const std::string& fp8_format) {
    const Fp8Args a = fp8_common(x, x_fp8, scale, fp8_format);
    expect_int("amax_scratch", amax_scratch, at::kInt, "int32");
    if (amax_scratch.numel() != 1)
        value_error("shape mismatch: amax_scratch must have exactly 1 element; got shape " + shape_str(amax_scratch));
    if (scale.numel() != 1)
        value_error("shape mismatch: scale must have exactly 1 element; got shape " + shape_str(scale));
    Launch l(x, {&x_fp8, &scale, &amax_scratch});
    check_launch("launch_fp8_quant_tensor_fwd",
                 launch_fp8_quant_tensor_fwd(x.data_ptr(), static_cast<uint8_t*>(x_fp8.data_ptr()),
                                             static_cast<float*>(scale.data_ptr()),
                                             static_cast<int32_t*>(amax_scratch.data_ptr()), a.m, a.n, a.dt, a.fmt,
                                             l.stream));
}

void fp8_quant_token_fwd(const at::Tensor& x, const at::Tensor& x_fp8, const at::Tensor& scale,
                         const std::string& fp8_format) {
    const Fp8Args a = fp8_common(x, x_fp8, scale, fp8_format);
    if (scale.numel() != a.m || scale.dim() < 1 || scale.size(0) != a.m)
        value_error("shape mismatch: scale shape " + shape_str(scale) + " must be [" + std::to_string(a.m) + ", 1]");
    Launch l(x, {&x_fp8, &scale});
    check_launch("launch_fp8_quant_token_fwd",
                 launch_fp8_quant_token_fwd(x.data_ptr(), static_cast<uint8_t*>(x_fp8.data_ptr()),
                                            static_cast<float*>(scale.data_ptr()), a.m, a.n, a.dt, a.fmt, l.stream));
}

// ------------------------------------------------------------------ src/kernels/matmul_add_bias.rs:36-122
void matmul_add_bias_fwd(const at::Tensor& x, const at::Tensor& weight, const c10::optional<at::Tensor>& bias,
                         const at::Tensor& y) {
    const int32_t dt = tag_of("x", x);
    expect_float_input("x", dt);
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    const bool has_bias = bias.has_value() && bias->defined();
    if (has_bias) expect_same_dtype("bias", tag_of("bias", *bias), dt);
    if (x.dim() != 2 || weight.dim() != 2)
        value_error("shape mismatch: x and weight must be 2-D; got x=" + shape_str(x) + ", weight=" + shape_str(weight));
    const int64_t m = x.size(0), k = x.size(1), n = weight.size(0);
    if (weight.size(1) != k)
        value_error("shape mismatch: weight's in_features (" + std::to_string(weight.size(1)) +
                    ") must match x's last dim (" + std::to_string(k) + ")");
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != n)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " +
                    std::to_string(n) + "]");
    if (has_bias && (bias->dim() != 1 || bias->size(0) != n))
        value_error("shape mismatch: bias shape " + shape_str(*bias) + " must be [" + std::to_string(n) + "]");
    at::Tensor none;
    Launch l(x, {&weight, &y, has_bias ? &*bias : &none});
    check_launch("launch_matmul_add_bias_fwd",
                 launch_matmul_add_bias_fwd(x.data_ptr(), weight.data_ptr(), has_bias ? bias->data_ptr() : nullptr,
                                            y.data_ptr(), m, k, n, dt, l.stream));
}

void matmul_add_bias_fp8_fwd(const at::Tensor& a, const at::Tensor& a_scale, const at::Tensor& w,
                             const at::Tensor& w_scale, const c10::optional<at::Tensor>& bias, const at::Tensor& y) {
    if (tag_of("a_fp8", a) != CCK_F8E4M3 || tag_of("w_fp8", w) != CCK_F8E4M3)
        value_error("unsupported dtype 'a_fp8 and w_fp8 must be float8_e4m3fn'");
    expect_f32("a_scale", tag_of("a_scale", a_scale));
    expect_f32("w_scale", tag_of("w_scale", w_scale));
    const int32_t odt = tag_of("y", y);
    if (odt != CCK_BF16 && odt != CCK_F16) value_error("unsupported dtype 'y must be bfloat16 or float16'");
    const bool has_bias = bias.has_value() && bias->defined();
    if (has_bias) expect_same_dtype("bias", tag_of("bias", *bias), odt);
    if (a.dim() != 2 || w.dim() != 2)
        value_error("shape mismatch: a_fp8 and w_fp8 must be 2-D; got a_fp8=" + shape_str(a) + ", w_fp8=" + shape_str(w));
    const int64_t m = a.size(0), k = a.size(1), n = w.size(0);
    if (w.size(1) != k)
        value_error("shape mismatch: w_fp8's in_features (" + std::to_string(w.size(1)) +
                    ") must match a_fp8's last dim (" + std::to_string(k) + ")");
    if (a_scale.numel() != m) value_error("shape mismatch: a_scale must have " + std::to_string(m) + " elements");
    if (w_scale.numel() != n) value_error("shape mismatch: w_scale must have " + std::to_string(n) + " elements");
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != n)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " +
                    std::to_string(n) + "]");
    if (has_bias && (bias->dim() != 1 || bias->size(0) != n))
        value_error("shape mismatch: bias shape " + shape_str(*bias) + " must be [" + std::to_string(n) + "]");
    at::Tensor none;
    Launch l(a, {&a_scale, &w, &w_scale, &y, has_bias ? &*bias : &none});
    check_launch("launch_matmul_add_bias_fp8_fwd",
                 launch_matmul_add_bias_fp8_fwd(static_cast<const uint8_t*>(a.data_ptr()),
                                                static_cast<const float*>(a_scale.data_ptr()),
                                                static_cast<const uint8_t*>(w.data_ptr()),
                                                static_cast<const float*>(w_scale.data_ptr()),
                                                has_bias ? bias->data_ptr() : nullptr, y.data_ptr(), m, k, n, odt,
                                                l.stream));
}

// fused epilogues (no counterpart in the reference)
void matmul_swiglu_fwd(const at::Tensor& x, const at::Tensor& w_gate_up, const at::Tensor& y) {
    const int32_t dt = tag_of("x", x);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "' for the fused path; expected float16 or bfloat16");
    expect_same_dtype("w_gate_up", tag_of("w_gate_up", w_gate_up), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    if (x.dim() != 2 || w_gate_up.dim() != 2)
        value_error("shape mismatch: x and w_gate_up must be 2-D; got x=" + shape_str(x) + ", w_gate_up=" + shape_str(w_gate_up));
    const int64_t m = x.size(0), k = x.size(1), f2 = w_gate_up.size(0);
    if (w_gate_up.size(1) != k)
        value_error("shape mismatch: w_gate_up's in_features (" + std::to_string(w_gate_up.size(1)) +
                    ") must match x's last dim (" + std::to_string(k) + ")");
    if (f2 % 256 != 0) value_error("shape mismatch: w_gate_up must have a multiple of 256 rows (128-feature gate/up blocks)");
    if (k % 8 != 0) value_error("shape mismatch: the fused path needs K to be a multiple of 8");
    const int64_t f = f2 / 2;
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != f)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " + std::to_string(f) + "]");
    Launch l(x, {&w_gate_up, &y});
    check_launch("launch_matmul_swiglu_fwd",
                 launch_matmul_swiglu_fwd(x.data_ptr(), w_gate_up.data_ptr(), y.data_ptr(), m, k, f, dt, l.stream));
}

void matmul_add_bias_residual_fwd(const at::Tensor& x, const at::Tensor& weight, const c10::optional<at::Tensor>& bias,
                                  const at::Tensor& residual, const at::Tensor& y) {
    const int32_t dt = tag_of("x", x);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "' for the fused path; expected float16 or bfloat16");
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("residual", tag_of("residual", residual), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    const bool has_bias = bias.has_value() && bias->defined();
    if (has_bias) expect_same_dtype("bias", tag_of("bias", *bias), dt);
    if (x.dim() != 2 || weight.dim() != 2)
        value_error("shape mismatch: x and weight must be 2-D; got x=" + shape_str(x) + ", weight=" + shape_str(weight));
    const int64_t m = x.size(0), k = x.size(1), n = weight.size(0);
    if (weight.size(1) != k)
        value_error("shape mismatch: weight's in_features (" + std::to_string(weight.size(1)) +
                    ") must match x's last dim (" + std::to_string(k) + ")");
    if (k % 8 != 0) value_error("shape mismatch: the fused path needs K to be a multiple of 8");
    for (const at::Tensor* t : {&residual, &y})
        if (t->dim() != 2 || t->size(0) != m || t->size(1) != n)
            value_error("shape mismatch: residual and y must be [" + std::to_string(m) + ", " + std::to_string(n) + "]");
    if (has_bias && (bias->dim() != 1 || bias->size(0) != n))
        value_error("shape mismatch: bias shape " + shape_str(*bias) + " must be [" + std::to_string(n) + "]");
    at::Tensor none;
    Launch l(x, {&weight, &residual, &y, has_bias ? &*bias : &none});
    check_launch("launch_matmul_add_bias_residual_fwd",
                 launch_matmul_add_bias_residual_fwd(x.data_ptr(), weight.data_ptr(), has_bias ? bias->data_ptr() : nullptr,
                                                     residual.data_ptr(), y.data_ptr(), m, k, n, dt, l.stream));
}

void matmul_add_bias_rope_fwd(const at::Tensor& x, const at::Tensor& weight, const c10::optional<at::Tensor>& bias,
                              const at::Tensor& cos, const at::Tensor& sin, const at::Tensor& y, int64_t rope_cols) {
    const int32_t dt = tag_of("x", x);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "' for the fused path; expected float16 or bfloat16");
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    expect_f32("cos", tag_of("cos", cos), " (RoPE tables are always fp32)");
    expect_f32("sin", tag_of("sin", sin), " (RoPE tables are always fp32)");
    const bool has_bias = bias.has_value() && bias->defined();
    if (has_bias) expect_same_dtype("bias", tag_of("bias", *bias), dt);
    if (x.dim() != 2 || weight.dim() != 2)
        value_error("shape mismatch: x and weight must be 2-D; got x=" + shape_str(x) + ", weight=" + shape_str(weight));
    const int64_t m = x.size(0), k = x.size(1), n = weight.size(0);
    if (weight.size(1) != k)
        value_error("shape mismatch: weight's in_features (" + std::to_string(weight.size(1)) +
                    ") must match x's last dim (" + std::to_string(k) + ")");
    if (k % 8 != 0) value_error("shape mismatch: the fused path needs K to be a multiple of 8");
    if (n % 128 != 0 || rope_cols % 128 != 0 || rope_cols < 0 || rope_cols > n)
        value_error("shape mismatch: heads are 128 columns wide: weight rows (" + std::to_string(n) + ") and rope_cols (" +
                    std::to_string(rope_cols) + ") must be multiples of 128 with rope_cols <= rows");
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != n)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " + std::to_string(n) + "]");
    if (cos.dim() != 2 || sin.dim() != 2 || cos.size(1) != 64 || sin.size(1) != 64 || cos.size(0) != sin.size(0) ||
        cos.size(0) < 1 || m % cos.size(0) != 0)
        value_error("shape mismatch: cos/sin must be [seq_len, 64] with x's rows (" + std::to_string(m) +
                    ") a multiple of seq_len; got cos=" + shape_str(cos) + ", sin=" + shape_str(sin));
    if (has_bias && (bias->dim() != 1 || bias->size(0) != n))
        value_error("shape mismatch: bias shape " + shape_str(*bias) + " must be [" + std::to_string(n) + "]");
    at::Tensor none;
    Launch l(x, {&weight, &cos, &sin, &y, has_bias ? &*bias : &none});
    check_launch("launch_matmul_add_bias_rope_fwd",
                 launch_matmul_add_bias_rope_fwd(x.data_ptr(), weight.data_ptr(), has_bias ? bias->data_ptr() : nullptr,
                                                 static_cast<const float*>(cos.data_ptr()),
                                                 static_cast<const float*>(sin.data_ptr()), y.data_ptr(), m, k, n,
                                                 rope_cols, cos.size(0), dt, l.stream));
}

// ------------------------------------------------------------------ src/kernels/linear_cross_entropy.rs:44-133
void linear_ce_chunk_update(const at::Tensor& logits_chunk, const at::Tensor& targets, int64_t v_start,
                            const at::Tensor& running_max, const at::Tensor& running_sum,
                            const at::Tensor& target_logit) {
    const int32_t dt = tag_of("logits_chunk", logits_chunk);
    expect_float_input("logits_chunk", dt);
    expect_int("targets", targets, at::kLong, "int64");
    expect_f32("running_max", tag_of("running_max", running_max));
    expect_f32("running_sum", tag_of("running_sum", running_sum));
    expect_f32("target_logit", tag_of("target_logit", target_logit));
    if (logits_chunk.dim() != 2)
        value_error("shape mismatch: logits_chunk must be 2-D [N, chunk_v], got " + shape_str(logits_chunk));
    const int64_t n = logits_chunk.size(0), chunk_v = logits_chunk.size(1);
    if (targets.dim() != 1 || targets.size(0) != n)
        value_error("shape mismatch: targets shape " + shape_str(targets) + " must be [" + std::to_string(n) +
                    "] (logits_chunk's row count)");
    const std::pair<const char*, const at::Tensor*> accs[] = {
        {"running_max", &running_max}, {"running_sum", &running_sum}, {"target_logit", &target_logit}};
    for (const auto& a : accs)
        if (a.second->dim() != 1 || a.second->size(0) != n)
            value_error(std::string("shape mismatch: ") + a.first + " shape " + shape_str(*a.second) + " must be [" +
                        std::to_string(n) + "]");
    Launch l(logits_chunk, {&targets, &running_max, &running_sum, &target_logit});
    check_launch("launch_linear_ce_chunk_update",
                 launch_linear_ce_chunk_update(logits_chunk.data_ptr(), static_cast<const int64_t*>(targets.data_ptr()),
                                               v_start, n, chunk_v, static_cast<float*>(running_max.data_ptr()),
                                               static_cast<float*>(running_sum.data_ptr()),
                                               static_cast<float*>(target_logit.data_ptr()), dt, l.stream));
}

// fused path (no counterpart in the reference)
void linear_cross_entropy_fwd(const at::Tensor& hidden, const at::Tensor& weight, const at::Tensor& targets,
                              int64_t v_start, const at::Tensor& row_stats, const at::Tensor& workspace,
                              const c10::optional<at::Tensor>& logits) {
    const int32_t dt = tag_of("hidden", hidden);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "' for the fused path; expected float16 or bfloat16");
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_int("targets", targets, at::kLong, "int64");
    expect_f32("row_stats", tag_of("row_stats", row_stats));
    check_cuda_contiguous("workspace", workspace);
    if (hidden.dim() != 2 || weight.dim() != 2)
        value_error("shape mismatch: hidden and weight must be 2-D; got hidden=" + shape_str(hidden) +
                    ", weight=" + shape_str(weight));
    const int64_t n = hidden.size(0), h = hidden.size(1), v = weight.size(0);
    if (weight.size(1) != h)
        value_error("shape mismatch: weight's hidden dim (" + std::to_string(weight.size(1)) +
                    ") must match hidden's last dim (" + std::to_string(h) + ")");
    if (targets.dim() != 1 || targets.size(0) != n)
        value_error("shape mismatch: targets shape " + shape_str(targets) + " must be [" + std::to_string(n) + "]");
    if (row_stats.dim() != 2 || row_stats.size(0) != 3 || row_stats.size(1) != n)
        value_error("shape mismatch: row_stats shape " + shape_str(row_stats) + " must be [3, " + std::to_string(n) + "]");
    if (h % 8 != 0) value_error("shape mismatch: the fused path needs hidden dim to be a multiple of 8");
    const int64_t ws_bytes = static_cast<int64_t>(workspace.numel()) * workspace.element_size();
    if (ws_bytes < cck_lce_workspace_bytes(n, v))
        value_error("shape mismatch: workspace has " + std::to_string(ws_bytes) + " bytes, needs " +
                    std::to_string(cck_lce_workspace_bytes(n, v)));
    if (logits.has_value()) {      // gradient path: also keep the fp32 logits
        const at::Tensor& lg = *logits;
        expect_f32("logits", tag_of("logits", lg));
        if (lg.dim() != 2 || lg.size(0) != n || lg.size(1) != v)
            value_error("shape mismatch: logits shape " + shape_str(lg) + " must be [" + std::to_string(n) + ", " +
                        std::to_string(v) + "]");
        if (v % 4 != 0) value_error("shape mismatch: storing the logits needs a vocabulary size that is a multiple of 4");
        Launch l(hidden, {&weight, &targets, &row_stats, &workspace, &lg});
        check_launch("launch_linear_cross_entropy_fwd_store",
                     launch_linear_cross_entropy_fwd_store(hidden.data_ptr(), weight.data_ptr(),
                                                           static_cast<const int64_t*>(targets.data_ptr()), v_start, n,
                                                           h, v, static_cast<float*>(row_stats.data_ptr()),
                                                           workspace.data_ptr(), ws_bytes,
                                                           static_cast<float*>(lg.data_ptr()), dt, l.stream));
        return;
    }
    Launch l(hidden, {&weight, &targets, &row_stats, &workspace});
    check_launch("launch_linear_cross_entropy_fwd",
                 launch_linear_cross_entropy_fwd(hidden.data_ptr(), weight.data_ptr(),
                                                 static_cast<const int64_t*>(targets.data_ptr()), v_start, n, h, v,
                                                 static_cast<float*>(row_stats.data_ptr()), workspace.data_ptr(),
                                                 ws_bytes, dt, l.stream));
}

// backward helpers (no counterpart in the reference)
void lce_dlogits_fwd(const at::Tensor& hidden, const at::Tensor& weight, const at::Tensor& targets,
                     const at::Tensor& lse, int64_t ignore_index, double grad_scale, const at::Tensor& dlogits) {
    const int32_t dt = tag_of("hidden", hidden);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "'; expected float16 or bfloat16");
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("dlogits", tag_of("dlogits", dlogits), dt);
    expect_int("targets", targets, at::kLong, "int64");
    expect_f32("lse", tag_of("lse", lse));
    if (hidden.dim() != 2 || weight.dim() != 2 || weight.size(1) != hidden.size(1))
        value_error("shape mismatch: hidden [N, H] and weight [V, H] expected; got hidden=" + shape_str(hidden) +
                    ", weight=" + shape_str(weight));
    const int64_t n = hidden.size(0), h = hidden.size(1), v = weight.size(0);
    if (targets.numel() != n || lse.numel() != n) value_error("shape mismatch: targets and lse must have " + std::to_string(n) + " elements");
    if (dlogits.dim() != 2 || dlogits.size(0) != n || dlogits.size(1) != v)
        value_error("shape mismatch: dlogits shape " + shape_str(dlogits) + " must be [" + std::to_string(n) + ", " + std::to_string(v) + "]");
    if (h % 8 != 0) value_error("shape mismatch: hidden dim must be a multiple of 8");
    Launch l(hidden, {&weight, &targets, &lse, &dlogits});
    check_launch("launch_lce_dlogits_fwd",
                 launch_lce_dlogits_fwd(hidden.data_ptr(), weight.data_ptr(), static_cast<const int64_t*>(targets.data_ptr()),
                                        static_cast<const float*>(lse.data_ptr()), n, h, v, ignore_index,
                                        static_cast<float>(grad_scale), dlogits.data_ptr(), dt, l.stream));
}

void lce_dlogits_from_logits(const at::Tensor& logits, const at::Tensor& targets, const at::Tensor& lse,
                             int64_t ignore_index, double grad_scale, const at::Tensor& dlogits,
                             const c10::optional<at::Tensor>& dlogits_t_opt) {
    const bool want_t = dlogits_t_opt.has_value() && dlogits_t_opt->defined();
    const at::Tensor dlogits_t = want_t ? *dlogits_t_opt : at::Tensor();
    expect_f32("logits", tag_of("logits", logits));
    expect_f32("lse", tag_of("lse", lse));
    expect_int("targets", targets, at::kLong, "int64");
    const int32_t dt = tag_of("dlogits", dlogits);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "'; expected float16 or bfloat16");
    // dlogits_t may be a column range of a wider row-major matrix (the transposes of several row
    // chunks side by side): rows are stride(0) apart, elements within a row adjacent
    if (want_t && !dlogits_t.is_cuda()) value_error("argument 'dlogits_t' must be a CUDA tensor");
    if (want_t && dlogits_t.scalar_type() != dlogits.scalar_type())
        value_error("dtype mismatch: 'dlogits_t' must have dlogits' dtype");
    if (logits.dim() != 2) value_error("shape mismatch: logits must be 2-D; got " + shape_str(logits));
    const int64_t n = logits.size(0), v = logits.size(1);
    if (targets.numel() != n || lse.numel() != n)
        value_error("shape mismatch: targets and lse must have " + std::to_string(n) + " elements");
    if (dlogits.dim() != 2 || dlogits.size(0) != n || dlogits.size(1) != v)
        value_error("shape mismatch: dlogits shape " + shape_str(dlogits) + " must be " + shape_str(logits));
    if (want_t && (dlogits_t.dim() != 2 || dlogits_t.size(0) != v || dlogits_t.size(1) < n || dlogits_t.stride(1) != 1 ||
        dlogits_t.stride(0) < dlogits_t.size(1) || dlogits_t.stride(0) % 4 != 0 || dlogits_t.storage_offset() % 4 != 0))
        value_error("shape mismatch: dlogits_t shape " + shape_str(dlogits_t) + " must be [" + std::to_string(v) +
                    ", >= " + std::to_string(n) + "] with unit inner stride, and a row pitch and offset that are multiples of 4");
    if (v % 4 != 0) value_error("shape mismatch: the vocabulary size must be a multiple of 4");
    Launch l(logits, {&targets, &lse, &dlogits, &dlogits_t});
    check_launch("launch_lce_dlogits_from_logits",
                 launch_lce_dlogits_from_logits(static_cast<const float*>(logits.data_ptr()),
                                                static_cast<const int64_t*>(targets.data_ptr()),
                                                static_cast<const float*>(lse.data_ptr()), n, v, ignore_index,
                                                static_cast<float>(grad_scale), dlogits.data_ptr(),
                                                want_t ? dlogits_t.data_ptr() : nullptr, want_t ? dlogits_t.stride(0) : 0,
                                                dt, l.stream));
}

void transpose_2byte(const at::Tensor& in, const at::Tensor& out) {
    const int32_t dt = tag_of("in", in);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "'; expected float16 or bfloat16");
    expect_same_dtype("out", tag_of("out", out), dt);
    if (in.dim() != 2 || out.dim() != 2 || out.size(0) != in.size(1) || out.size(1) < in.size(0))
        value_error("shape mismatch: in [R, C] and out [C, >= R] expected; got in=" + shape_str(in) + ", out=" + shape_str(out));
    if (in.size(1) % 4 != 0 || out.size(1) % 4 != 0)
        value_error("shape mismatch: in's columns and out's row length must be multiples of 4");
    Launch l(in, {&out});
    check_launch("launch_transpose_2byte",
                 launch_transpose_2byte(in.data_ptr(), in.size(0), in.size(1), out.data_ptr(), out.size(1), l.stream));
}

void matmul_accumulate_f32_fwd(const at::Tensor& x, const at::Tensor& weight, const at::Tensor& y) {
    const int32_t dt = tag_of("x", x);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "'; expected float16 or bfloat16");
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_f32("y", tag_of("y", y));
    if (x.dim() != 2 || weight.dim() != 2 || weight.size(1) != x.size(1))
        value_error("shape mismatch: x [M, K] and weight [N, K] expected; got x=" + shape_str(x) + ", weight=" + shape_str(weight));
    const int64_t m = x.size(0), k = x.size(1), n = weight.size(0);
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != n)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " + std::to_string(n) + "]");
    if (k % 8 != 0) value_error("shape mismatch: K must be a multiple of 8");
    Launch l(x, {&weight, &y});
    check_launch("launch_matmul_accumulate_f32_fwd",
                 launch_matmul_accumulate_f32_fwd(x.data_ptr(), weight.data_ptr(), static_cast<float*>(y.data_ptr()), m, k,
                                                  n, dt, l.stream));
}

int64_t lce_workspace_bytes(const at::Tensor& like, int64_t n, int64_t v) {
    c10::cuda::CUDAGuard guard(like.device());
    return cck_lce_workspace_bytes(n, v);
}

void lce_finalize(const at::Tensor& stats, const at::Tensor& targets, int64_t ignore_index,
                  const c10::optional<at::Tensor>& loss_rows, const at::Tensor& reduce_out) {
    expect_f32("stats", tag_of("stats", stats));
    expect_int("targets", targets, at::kLong, "int64");
    expect_f32("reduce_out", tag_of("reduce_out", reduce_out));
    const int64_t n = targets.numel();
    if (stats.dim() != 3 || stats.size(1) != 3 || stats.size(2) != n || stats.size(0) < 1)
        value_error("shape mismatch: stats shape " + shape_str(stats) + " must be [shards, 3, " + std::to_string(n) + "]");
    if (reduce_out.numel() != 2) value_error("shape mismatch: reduce_out must have 2 elements");
    const bool want_rows = loss_rows.has_value() && loss_rows->defined();
    if (want_rows) {
        expect_f32("loss_rows", tag_of("loss_rows", *loss_rows));
        if (loss_rows->numel() != n) value_error("shape mismatch: loss_rows must have " + std::to_string(n) + " elements");
    }
    at::Tensor none;
    Launch l(stats, {&targets, &reduce_out, want_rows ? &*loss_rows : &none});
    check_launch("launch_lce_finalize",
                 launch_lce_finalize(static_cast<const float*>(stats.data_ptr()),
                                     static_cast<const int64_t*>(targets.data_ptr()), n, stats.size(0), ignore_index,
                                     want_rows ? static_cast<float*>(loss_rows->data_ptr()) : nullptr,
                                     static_cast<float*>(reduce_out.data_ptr()), l.stream));
}

uint32_t take_device_status(const at::Tensor& like) {
    c10::cuda::CUDAGuard guard(like.device());
    uint32_t v = 0;
    check_launch("cck_take_device_status", cck_take_device_status(&v));
    return v;
}

// GEMM (+ bias, + residual) that also leaves per-(row, 256-column tile) statistics of its output
void matmul_add_bias_stats_fwd(const at::Tensor& x, const at::Tensor& weight, const c10::optional<at::Tensor>& bias,
                               const c10::optional<at::Tensor>& residual, const at::Tensor& y,
                               const c10::optional<at::Tensor>& row_sumsq, const c10::optional<at::Tensor>& row_amax) {
    const int32_t dt = tag_of("x", x);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "' for the fused path; expected float16 or bfloat16");
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    const bool has_bias = bias.has_value() && bias->defined();
    const bool has_res = residual.has_value() && residual->defined();
    if (has_bias) expect_same_dtype("bias", tag_of("bias", *bias), dt);
    if (has_res) expect_same_dtype("residual", tag_of("residual", *residual), dt);
    if (x.dim() != 2 || weight.dim() != 2)
        value_error("shape mismatch: x and weight must be 2-D; got x=" + shape_str(x) + ", weight=" + shape_str(weight));
    const int64_t m = x.size(0), k = x.size(1), n = weight.size(0);
    if (weight.size(1) != k)
        value_error("shape mismatch: weight's in_features (" + std::to_string(weight.size(1)) +
                    ") must match x's last dim (" + std::to_string(k) + ")");
    if (k % 8 != 0) value_error("shape mismatch: the fused path needs K to be a multiple of 8");
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != n)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " + std::to_string(n) + "]");
    if (has_bias && (bias->dim() != 1 || bias->size(0) != n))
        value_error("shape mismatch: bias shape " + shape_str(*bias) + " must be [" + std::to_string(n) + "]");
    if (has_res && residual->sizes() != y.sizes())
        value_error("shape mismatch: residual shape " + shape_str(*residual) + " must match y's " + shape_str(y));
    const int64_t tiles = cck_gemm_stat_tiles(n);
    at::Tensor none;
    const at::Tensor* stats[2] = {row_sumsq.has_value() && row_sumsq->defined() ? &*row_sumsq : nullptr,
                                  row_amax.has_value() && row_amax->defined() ? &*row_amax : nullptr};
    const char* stat_names[2] = {"row_sumsq", "row_amax"};
    for (int i = 0; i < 2; ++i) {
        if (!stats[i]) continue;
        expect_f32(stat_names[i], tag_of(stat_names[i], *stats[i]));
        if (stats[i]->dim() != 2 || stats[i]->size(0) != tiles || stats[i]->size(1) != m)
            value_error(std::string("shape mismatch: ") + stat_names[i] + " shape " + shape_str(*stats[i]) + " must be [" +
                        std::to_string(tiles) + ", " + std::to_string(m) + "]");
    }
    Launch l(x, {&weight, &y, has_bias ? &*bias : &none, has_res ? &*residual : &none, stats[0] ? stats[0] : &none,
                 stats[1] ? stats[1] : &none});
    check_launch("launch_matmul_add_bias_stats_fwd",
                 launch_matmul_add_bias_stats_fwd(x.data_ptr(), weight.data_ptr(), has_bias ? bias->data_ptr() : nullptr,
                                                  has_res ? residual->data_ptr() : nullptr, y.data_ptr(),
                                                  stats[0] ? static_cast<float*>(stats[0]->data_ptr()) : nullptr,
                                                  stats[1] ? static_cast<float*>(stats[1]->data_ptr()) : nullptr, m, k, n, dt,
                                                  l.stream));
}

void rmsnorm_from_stats_fwd(const at::Tensor& x, const at::Tensor& row_sumsq, const at::Tensor& weight,
                            const at::Tensor& y, double eps) {
    const int32_t dt = tag_of("x", x);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "'; expected float16 or bfloat16");
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    expect_same_dtype("y", tag_of("y", y), dt);
    expect_f32("row_sumsq", tag_of("row_sumsq", row_sumsq));
    if (x.dim() != 2 || y.sizes() != x.sizes())
        value_error("shape mismatch: x and y must be 2-D of the same shape; got x=" + shape_str(x) + ", y=" + shape_str(y));
    const int64_t rows = x.size(0), cols = x.size(1);
    if (weight.dim() != 1 || weight.size(0) != cols)
        value_error("shape mismatch: weight shape " + shape_str(weight) + " must be [" + std::to_string(cols) + "]");
    if (row_sumsq.dim() != 2 || row_sumsq.size(1) != rows || row_sumsq.size(0) < 1)
        value_error("shape mismatch: row_sumsq shape " + shape_str(row_sumsq) + " must be [n_tiles, " + std::to_string(rows) + "]");
    if (cols % 8 != 0) value_error("shape mismatch: cols must be a multiple of 8");
    Launch l(x, {&row_sumsq, &weight, &y});
    check_launch("launch_rmsnorm_from_stats_fwd",
                 launch_rmsnorm_from_stats_fwd(x.data_ptr(), static_cast<const float*>(row_sumsq.data_ptr()),
                                               row_sumsq.size(0), weight.data_ptr(), y.data_ptr(), rows, cols,
                                               static_cast<float>(eps), dt, l.stream));
}

void fp8_quant_token_from_amax_fwd(const at::Tensor& x, const at::Tensor& row_amax, const at::Tensor& x_fp8,
                                   const at::Tensor& scale, const std::string& fp8_format) {
    const int32_t dt = tag_of("x", x);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "'; expected float16 or bfloat16");
    const int32_t fmt = parse_fp8_format(fp8_format);
    if (tag_of("x_fp8", x_fp8) != fmt) value_error("dtype mismatch: x_fp8 must be the torch float8 type of fp8_format");
    expect_f32("scale", tag_of("scale", scale));
    expect_f32("row_amax", tag_of("row_amax", row_amax));
    if (x.dim() != 2 || x_fp8.sizes() != x.sizes())
        value_error("shape mismatch: x and x_fp8 must be 2-D of the same shape; got x=" + shape_str(x) + ", x_fp8=" + shape_str(x_fp8));
    const int64_t m = x.size(0), n = x.size(1);
    if (scale.numel() != m) value_error("shape mismatch: scale must have " + std::to_string(m) + " elements");
    if (row_amax.dim() != 2 || row_amax.size(1) != m || row_amax.size(0) < 1)
        value_error("shape mismatch: row_amax shape " + shape_str(row_amax) + " must be [n_tiles, " + std::to_string(m) + "]");
    if (n % 8 != 0) value_error("shape mismatch: n must be a multiple of 8");
    Launch l(x, {&row_amax, &x_fp8, &scale});
    check_launch("launch_fp8_quant_token_from_amax_fwd",
                 launch_fp8_quant_token_from_amax_fwd(x.data_ptr(), static_cast<const float*>(row_amax.data_ptr()),
                                                      row_amax.size(0), static_cast<uint8_t*>(x_fp8.data_ptr()),
                                                      static_cast<float*>(scale.data_ptr()), m, n, dt, fmt, l.stream));
}

// rmsnorm -> per-token FP8 quantisation in one pass
void rmsnorm_fp8_quant_token_fwd(const at::Tensor& x, const at::Tensor& weight, const c10::optional<at::Tensor>& row_sumsq,
                                 const c10::optional<at::Tensor>& y, const at::Tensor& x_fp8, const at::Tensor& scale,
                                 double eps, const std::string& fp8_format) {
    const int32_t dt = tag_of("x", x);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "'; expected float16 or bfloat16");
    expect_same_dtype("weight", tag_of("weight", weight), dt);
    const int32_t fmt = parse_fp8_format(fp8_format);
    if (tag_of("x_fp8", x_fp8) != fmt) value_error("dtype mismatch: x_fp8 must be the torch float8 type of fp8_format");
    expect_f32("scale", tag_of("scale", scale));
    if (x.dim() != 2 || x_fp8.sizes() != x.sizes())
        value_error("shape mismatch: x and x_fp8 must be 2-D of the same shape; got x=" + shape_str(x) + ", x_fp8=" + shape_str(x_fp8));
    const int64_t rows = x.size(0), cols = x.size(1);
    if (weight.dim() != 1 || weight.size(0) != cols)
        value_error("shape mismatch: weight shape " + shape_str(weight) + " must be [" + std::to_string(cols) + "]");
    if (scale.numel() != rows) value_error("shape mismatch: scale must have " + std::to_string(rows) + " elements");
    if (cols % 8 != 0) value_error("shape mismatch: cols must be a multiple of 8");
    const bool has_ss = row_sumsq.has_value() && row_sumsq->defined();
    const bool has_y = y.has_value() && y->defined();
    if (has_ss) {
        expect_f32("row_sumsq", tag_of("row_sumsq", *row_sumsq));
        if (row_sumsq->dim() != 2 || row_sumsq->size(1) != rows || row_sumsq->size(0) < 1)
            value_error("shape mismatch: row_sumsq shape " + shape_str(*row_sumsq) + " must be [n_tiles, " + std::to_string(rows) + "]");
    }
    if (has_y) {
        expect_same_dtype("y", tag_of("y", *y), dt);
        if (y->sizes() != x.sizes()) value_error("shape mismatch: y shape " + shape_str(*y) + " must match x's " + shape_str(x));
    }
    at::Tensor none;
    Launch l(x, {&weight, &x_fp8, &scale, has_ss ? &*row_sumsq : &none, has_y ? &*y : &none});
    check_launch("launch_rmsnorm_fp8_quant_token_fwd",
                 launch_rmsnorm_fp8_quant_token_fwd(x.data_ptr(), weight.data_ptr(),
                                                    has_ss ? static_cast<const float*>(row_sumsq->data_ptr()) : nullptr,
                                                    has_ss ? row_sumsq->size(0) : 0, has_y ? y->data_ptr() : nullptr,
                                                    static_cast<uint8_t*>(x_fp8.data_ptr()), static_cast<float*>(scale.data_ptr()),
                                                    rows, cols, static_cast<float>(eps), dt, fmt, l.stream));
}

// shared checks of the FP8 GEMM entry points; returns (m, k, n)
std::tuple<int64_t, int64_t, int64_t> check_fp8_operands(const at::Tensor& a, const at::Tensor& a_scale, const at::Tensor& w,
                                                         const at::Tensor& w_scale) {
    if (tag_of("a_fp8", a) != CCK_F8E4M3 || tag_of("w_fp8", w) != CCK_F8E4M3)
        value_error("unsupported dtype 'a_fp8 and w_fp8 must be float8_e4m3fn'");
    expect_f32("a_scale", tag_of("a_scale", a_scale));
    expect_f32("w_scale", tag_of("w_scale", w_scale));
    if (a.dim() != 2 || w.dim() != 2)
        value_error("shape mismatch: a_fp8 and w_fp8 must be 2-D; got a_fp8=" + shape_str(a) + ", w_fp8=" + shape_str(w));
    const int64_t m = a.size(0), k = a.size(1), n = w.size(0);
    if (w.size(1) != k)
        value_error("shape mismatch: w_fp8's in_features (" + std::to_string(w.size(1)) + ") must match a_fp8's last dim (" +
                    std::to_string(k) + ")");
    if (a_scale.numel() != m) value_error("shape mismatch: a_scale must have " + std::to_string(m) + " elements");
    if (w_scale.numel() != n) value_error("shape mismatch: w_scale must have " + std::to_string(n) + " elements");
    if (k % 16 != 0) value_error("shape mismatch: the fused FP8 GEMMs need K to be a multiple of 16, got " + std::to_string(k));
    return {m, k, n};
}

void matmul_swiglu_fp8_fwd(const at::Tensor& a, const at::Tensor& a_scale, const at::Tensor& w_gate_up,
                           const at::Tensor& w_scale, const at::Tensor& y, const c10::optional<at::Tensor>& row_amax) {
    auto [m, k, f2] = check_fp8_operands(a, a_scale, w_gate_up, w_scale);
    const int32_t odt = tag_of("y", y);
    if (odt != CCK_BF16 && odt != CCK_F16) value_error("unsupported dtype 'y must be bfloat16 or float16'");
    if (f2 % 256 != 0) value_error("shape mismatch: w_gate_up must have a multiple of 256 rows (128-feature gate/up blocks)");
    const int64_t f = f2 / 2;
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != f)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " + std::to_string(f) + "]");
    const bool has_amax = row_amax.has_value() && row_amax->defined();
    if (has_amax) {
        expect_f32("row_amax", tag_of("row_amax", *row_amax));
        if (row_amax->dim() != 2 || row_amax->size(0) != f / 128 || row_amax->size(1) != m)
            value_error("shape mismatch: row_amax shape " + shape_str(*row_amax) + " must be [" + std::to_string(f / 128) + ", " +
                        std::to_string(m) + "]");
    }
    at::Tensor none;
    Launch l(a, {&a_scale, &w_gate_up, &w_scale, &y, has_amax ? &*row_amax : &none});
    check_launch("launch_matmul_swiglu_fp8_fwd",
                 launch_matmul_swiglu_fp8_fwd(static_cast<const uint8_t*>(a.data_ptr()), static_cast<const float*>(a_scale.data_ptr()),
                                              static_cast<const uint8_t*>(w_gate_up.data_ptr()),
                                              static_cast<const float*>(w_scale.data_ptr()), y.data_ptr(),
                                              has_amax ? static_cast<float*>(row_amax->data_ptr()) : nullptr, m, k, f, odt,
                                              l.stream));
}

void matmul_add_bias_residual_fp8_fwd(const at::Tensor& a, const at::Tensor& a_scale, const at::Tensor& w,
                                      const at::Tensor& w_scale, const c10::optional<at::Tensor>& bias,
                                      const at::Tensor& residual, const at::Tensor& y) {
    auto [m, k, n] = check_fp8_operands(a, a_scale, w, w_scale);
    const int32_t odt = tag_of("y", y);
    if (odt != CCK_BF16 && odt != CCK_F16) value_error("unsupported dtype 'y must be bfloat16 or float16'");
    expect_same_dtype("residual", tag_of("residual", residual), odt);
    const bool has_bias = bias.has_value() && bias->defined();
    if (has_bias) expect_same_dtype("bias", tag_of("bias", *bias), odt);
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != n)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " + std::to_string(n) + "]");
    if (residual.sizes() != y.sizes())
        value_error("shape mismatch: residual shape " + shape_str(residual) + " must match y's " + shape_str(y));
    if (has_bias && (bias->dim() != 1 || bias->size(0) != n))
        value_error("shape mismatch: bias shape " + shape_str(*bias) + " must be [" + std::to_string(n) + "]");
    at::Tensor none;
    Launch l(a, {&a_scale, &w, &w_scale, &residual, &y, has_bias ? &*bias : &none});
    check_launch("launch_matmul_add_bias_residual_fp8_fwd",
                 launch_matmul_add_bias_residual_fp8_fwd(static_cast<const uint8_t*>(a.data_ptr()),
                                                         static_cast<const float*>(a_scale.data_ptr()),
                                                         static_cast<const uint8_t*>(w.data_ptr()),
                                                         static_cast<const float*>(w_scale.data_ptr()),
                                                         has_bias ? bias->data_ptr() : nullptr, residual.data_ptr(), y.data_ptr(),
                                                         m, k, n, odt, l.stream));
}

void matmul_add_bias_rope_fp8_fwd(const at::Tensor& a, const at::Tensor& a_scale, const at::Tensor& w,
                                  const at::Tensor& w_scale, const c10::optional<at::Tensor>& bias, const at::Tensor& cos,
                                  const at::Tensor& sin, const at::Tensor& y, int64_t rope_cols) {
    auto [m, k, n] = check_fp8_operands(a, a_scale, w, w_scale);
    const int32_t odt = tag_of("y", y);
    if (odt != CCK_BF16 && odt != CCK_F16) value_error("unsupported dtype 'y must be bfloat16 or float16'");
    expect_f32("cos", tag_of("cos", cos), " (RoPE tables are always fp32)");
    expect_f32("sin", tag_of("sin", sin), " (RoPE tables are always fp32)");
    const bool has_bias = bias.has_value() && bias->defined();
    if (has_bias) expect_same_dtype("bias", tag_of("bias", *bias), odt);
    if (k % 16 != 0) value_error("shape mismatch: the fused FP8 path needs K to be a multiple of 16");
    if (n % 128 != 0 || rope_cols % 128 != 0 || rope_cols < 0 || rope_cols > n)
        value_error("shape mismatch: heads are 128 columns wide: weight rows (" + std::to_string(n) + ") and rope_cols (" +
                    std::to_string(rope_cols) + ") must be multiples of 128 with rope_cols <= rows");
    if (y.dim() != 2 || y.size(0) != m || y.size(1) != n)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " + std::to_string(n) + "]");
    if (cos.dim() != 2 || sin.dim() != 2 || cos.size(1) != 64 || sin.size(1) != 64 || cos.size(0) != sin.size(0) ||
        cos.size(0) < 1 || m % cos.size(0) != 0)
        value_error("shape mismatch: cos/sin must be [seq_len, 64] with the rows of a_fp8 (" + std::to_string(m) +
                    ") a multiple of seq_len; got cos=" + shape_str(cos) + ", sin=" + shape_str(sin));
    if (has_bias && (bias->dim() != 1 || bias->size(0) != n))
        value_error("shape mismatch: bias shape " + shape_str(*bias) + " must be [" + std::to_string(n) + "]");
    at::Tensor none;
    Launch l(a, {&a_scale, &w, &w_scale, &cos, &sin, &y, has_bias ? &*bias : &none});
    check_launch("launch_matmul_add_bias_rope_fp8_fwd",
                 launch_matmul_add_bias_rope_fp8_fwd(static_cast<const uint8_t*>(a.data_ptr()),
                                                     static_cast<const float*>(a_scale.data_ptr()),
                                                     static_cast<const uint8_t*>(w.data_ptr()),
                                                     static_cast<const float*>(w_scale.data_ptr()),
                                                     has_bias ? bias->data_ptr() : nullptr,
                                                     static_cast<const float*>(cos.data_ptr()),
                                                     static_cast<const float*>(sin.data_ptr()), y.data_ptr(), m, k, n,
                                                     rope_cols, cos.size(0), odt, l.stream));
}

// y = op(a) op(b)^T with operands read as stored (transposed or not); see launch_matmul_general_fwd
void matmul_general_fwd(const at::Tensor& a, const at::Tensor& b, const at::Tensor& y, bool a_is_km, bool b_is_kn,
                        bool accumulate) {
    const int32_t dt = tag_of("a", a);
    if (dt != CCK_BF16 && dt != CCK_F16)
        value_error(std::string("unsupported dtype '") + tag_name(dt) + "'; expected float16 or bfloat16");
    expect_same_dtype("b", tag_of("b", b), dt);
    const int32_t ydt = tag_of("y", y);
    if (accumulate) expect_f32("y", ydt, " when accumulating");
    else expect_same_dtype("y", ydt, dt);
    if (a.dim() != 2 || b.dim() != 2 || y.dim() != 2) value_error("shape mismatch: a, b and y must be 2-D");
    const int64_t m = a_is_km ? a.size(1) : a.size(0), k = a_is_km ? a.size(0) : a.size(1);
    const int64_t n = b_is_kn ? b.size(1) : b.size(0), kb = b_is_kn ? b.size(0) : b.size(1);
    if (kb != k)
        value_error("shape mismatch: contraction lengths differ: a gives " + std::to_string(k) + ", b gives " + std::to_string(kb));
    if (y.size(0) != m || y.size(1) != n)
        value_error("shape mismatch: y shape " + shape_str(y) + " must be [" + std::to_string(m) + ", " + std::to_string(n) + "]");
    if (a.size(1) % 8 != 0 || b.size(1) % 8 != 0)
        value_error("shape mismatch: the contiguous dimension of a and of b must be a multiple of 8");
    Launch l(a, {&b, &y});
    check_launch("launch_matmul_general_fwd",
                 launch_matmul_general_fwd(a.data_ptr(), b.data_ptr(), y.data_ptr(), m, k, n, a_is_km ? 1 : 0,
                                           b_is_kn ? 1 : 0, accumulate ? 1 : 0, dt, l.stream));
}

uint64_t set_wait_limit_ns(const at::Tensor& like, uint64_t limit_ns) {
    c10::cuda::CUDAGuard guard(like.device());
    uint64_t previous = 0;
    check_launch("cck_set_wait_limit_ns", cck_set_wait_limit_ns(limit_ns, &previous));
    return previous;
}

void wait_limit_selftest(const at::Tensor& a, const at::Tensor& b, const at::Tensor& y, int64_t variant) {
    for (const auto& named : {std::make_pair("a", &a), std::make_pair("b", &b), std::make_pair("y", &y)})
        if (tag_of(named.first, *named.second) != CCK_BF16)
            value_error(std::string("unsupported dtype '") + named.first + " must be bfloat16'");
    if (a.numel() < 256 * 64 || b.numel() < 256 * 64 || y.numel() < 256 * 256)
        value_error("shape mismatch: a and b need 256 x 64 elements, y 256 x 256");
    if (variant < 0 || variant > 2) value_error("variant must be 0 (single CTA), 1 (CTA pair) or 2 (split-K cluster)");
    Launch l(a, {&b, &y});
    check_launch("launch_wait_limit_selftest",
                 launch_wait_limit_selftest(a.data_ptr(), b.data_ptr(), y.data_ptr(), static_cast<int32_t>(variant), l.stream));
}

}  // namespace

PYBIND11_MODULE(_native, m) {
    m.doc() = "validation + FFI layer over libcustom_cuda_b200 (C ABI in include/custom_cuda_b200.h)";
    m.def("rmsnorm_residual_fwd", &rmsnorm_residual_fwd, py::arg("x"), py::arg("residual"), py::arg("weight"),
          py::arg("y"), py::arg("residual_out"), py::arg("eps"));
    m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("weight"), py::arg("y"), py::arg("eps"));
    m.def("swiglu_fwd", &swiglu_fwd, py::arg("gate"), py::arg("up"), py::arg("y"));
    m.def("rope_fwd", &rope_fwd, py::arg("q"), py::arg("k"), py::arg("cos"), py::arg("sin"), py::arg("q_out"),
          py::arg("k_out"));
    m.def("linear_ce_chunk_update", &linear_ce_chunk_update, py::arg("logits_chunk"), py::arg("targets"),
          py::arg("v_start"), py::arg("running_max"), py::arg("running_sum"), py::arg("target_logit"));
    m.def("matmul_add_bias_fwd", &matmul_add_bias_fwd, py::arg("x"), py::arg("weight"), py::arg("bias").none(true),
          py::arg("y"));
    m.def("fp8_quant_block_fwd", &fp8_quant_block_fwd, py::arg("x"), py::arg("x_fp8"), py::arg("scale"),
          py::arg("fp8_format"));
    m.def("fp8_quant_tensor_fwd", &fp8_quant_tensor_fwd, py::arg("x"), py::arg("x_fp8"), py::arg("scale"),
          py::arg("amax_scratch"), py::arg("fp8_format"));
    // additions
    m.def("fp8_quant_token_fwd", &fp8_quant_token_fwd, py::arg("x"), py::arg("x_fp8"), py::arg("scale"),
          py::arg("fp8_format"));
    m.def("matmul_add_bias_fp8_fwd", &matmul_add_bias_fp8_fwd, py::arg("a_fp8"), py::arg("a_scale"), py::arg("w_fp8"),
          py::arg("w_scale"), py::arg("bias").none(true), py::arg("y"));
    m.def("rope_strided_fwd", &rope_strided_fwd, py::arg("q"), py::arg("k"), py::arg("cos"), py::arg("sin"),
          py::arg("q_out"), py::arg("k_out"));
    m.def("matmul_swiglu_fwd", &matmul_swiglu_fwd, py::arg("x"), py::arg("w_gate_up"), py::arg("y"));
    m.def("matmul_add_bias_rope_fwd", &matmul_add_bias_rope_fwd, py::arg("x"), py::arg("weight"),
          py::arg("bias").none(true), py::arg("cos"), py::arg("sin"), py::arg("y"), py::arg("rope_cols"));
    m.def("matmul_add_bias_residual_fwd", &matmul_add_bias_residual_fwd, py::arg("x"), py::arg("weight"),
          py::arg("bias").none(true), py::arg("residual"), py::arg("y"));
    m.def("linear_cross_entropy_fwd", &linear_cross_entropy_fwd, py::arg("hidden"), py::arg("weight"),
          py::arg("targets"), py::arg("v_start"), py::arg("row_stats"), py::arg("workspace"),
          py::arg("logits") = py::none());
    m.def("lce_dlogits_from_logits", &lce_dlogits_from_logits, py::arg("logits"), py::arg("targets"), py::arg("lse"),
          py::arg("ignore_index"), py::arg("grad_scale"), py::arg("dlogits"), py::arg("dlogits_t").none(true));
    m.def("lce_dlogits_fwd", &lce_dlogits_fwd, py::arg("hidden"), py::arg("weight"), py::arg("targets"), py::arg("lse"),
          py::arg("ignore_index"), py::arg("grad_scale"), py::arg("dlogits"));
    m.def("moe_router_fwd", &moe_router_fwd, py::arg("logits"), py::arg("topk_weights"), py::arg("topk_indices"),
          py::arg("renormalize"));
    m.def("token_gather_fwd", &token_gather_fwd, py::arg("src"), py::arg("indices"), py::arg("dst"));
    m.def("token_combine_fwd", &token_combine_fwd, py::arg("expert_output"), py::arg("unpermute_index"),
          py::arg("weights"), py::arg("combined"));
    m.def("token_dispatch_fwd", &token_dispatch_fwd, py::arg("src"), py::arg("src_row"), py::arg("dst_rank"),
          py::arg("dst_row"), py::arg("dst_bases"), py::arg("capacity_rows"));
    m.def("ep_plan", &ep_plan, py::arg("topk"), py::arg("counts"), py::arg("rank"), py::arg("src_row"), py::arg("dst_rank"),
          py::arg("dst_row"), py::arg("pull_rank"), py::arg("pull_row"), py::arg("meta"));
    m.def("token_combine_remote_fwd", &token_combine_remote_fwd, py::arg("src_bases"), py::arg("capacity_rows"),
          py::arg("src_rank"), py::arg("src_row"), py::arg("weights"), py::arg("combined"));
    m.def("swiglu_bwd", &swiglu_bwd, py::arg("gate"), py::arg("up"), py::arg("dy"), py::arg("dgate"), py::arg("dup"));
    m.def("rmsnorm_residual_bwd", &rmsnorm_residual_bwd, py::arg("dy"), py::arg("d_residual_out"),
          py::arg("residual_out"), py::arg("weight"), py::arg("dx"), py::arg("dweight"), py::arg("workspace"),
          py::arg("eps"));
    m.def("rmsnorm_bwd_workspace_bytes", &rmsnorm_bwd_workspace_bytes, py::arg("rows"), py::arg("cols"));
    m.def("transpose_2byte", &transpose_2byte, py::arg("input"), py::arg("out"));
    m.def("matmul_accumulate_f32_fwd", &matmul_accumulate_f32_fwd, py::arg("x"), py::arg("weight"), py::arg("y"));
    m.def("lce_workspace_bytes", &lce_workspace_bytes, py::arg("like"), py::arg("n"), py::arg("v_count"));
    m.def("lce_finalize", &lce_finalize, py::arg("stats"), py::arg("targets"), py::arg("ignore_index"),
          py::arg("loss_rows").none(true), py::arg("reduce_out"));
    m.def("matmul_add_bias_stats_fwd", &matmul_add_bias_stats_fwd, py::arg("x"), py::arg("weight"),
          py::arg("bias").none(true), py::arg("residual").none(true), py::arg("y"), py::arg("row_sumsq").none(true),
          py::arg("row_amax").none(true));
    m.def("rmsnorm_from_stats_fwd", &rmsnorm_from_stats_fwd, py::arg("x"), py::arg("row_sumsq"), py::arg("weight"),
          py::arg("y"), py::arg("eps"));
    m.def("fp8_quant_token_from_amax_fwd", &fp8_quant_token_from_amax_fwd, py::arg("x"), py::arg("row_amax"),
          py::arg("x_fp8"), py::arg("scale"), py::arg("fp8_format"));
    m.def("rmsnorm_fp8_quant_token_fwd", &rmsnorm_fp8_quant_token_fwd, py::arg("x"), py::arg("weight"),
          py::arg("row_sumsq").none(true), py::arg("y").none(true), py::arg("x_fp8"), py::arg("scale"), py::arg("eps"),
          py::arg("fp8_format"));
    m.def("matmul_swiglu_fp8_fwd", &matmul_swiglu_fp8_fwd, py::arg("a_fp8"), py::arg("a_scale"), py::arg("w_gate_up"),
          py::arg("w_scale"), py::arg("y"), py::arg("row_amax").none(true));
    m.def("matmul_add_bias_residual_fp8_fwd", &matmul_add_bias_residual_fp8_fwd, py::arg("a_fp8"), py::arg("a_scale"),
          py::arg("w_fp8"), py::arg("w_scale"), py::arg("bias").none(true), py::arg("residual"), py::arg("y"));
    m.def("matmul_add_bias_rope_fp8_fwd", &matmul_add_bias_rope_fp8_fwd, py::arg("a_fp8"), py::arg("a_scale"),
          py::arg("w_fp8"), py::arg("w_scale"), py::arg("bias").none(true), py::arg("cos"), py::arg("sin"), py::arg("y"),
          py::arg("rope_cols"));
    m.def("matmul_general_fwd", &matmul_general_fwd, py::arg("a"), py::arg("b"), py::arg("y"), py::arg("a_is_km"),
          py::arg("b_is_kn"), py::arg("accumulate"));
    m.def("gemm_stat_tiles", [](int64_t n) { return cck_gemm_stat_tiles(n); }, py::arg("n"));
    m.def("take_device_status", &take_device_status, py::arg("like"));
    m.def("set_wait_limit_ns", &set_wait_limit_ns, py::arg("like"), py::arg("limit_ns"));
    m.def("wait_limit_selftest", &wait_limit_selftest, py::arg("a"), py::arg("b"), py::arg("y"), py::arg("variant"));
}
