// The PyTorch extension module `mla_bwd_cuda`: the operator surface of the reference
// (`mla_bwd(q, kv, dO, lse, O, indices) -> (dQ, dKV)`, mla_bwd/mla_bwd.cu:972-1063) over the C ABI of
// include/smla_bwd.h.  This file only checks tensors, owns memory and picks the stream; every kernel
// lives behind the C ABI (smla_api.cu, compiled into the same module).
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <map>
#include <mutex>
#include <optional>
#include <tuple>

#include "../../include/smla_bwd.h"

namespace {

// Scratch kept per (device, stream) so that the six-argument call does not allocate gigabytes every time
// (the reference allocates only its small delta buffer per call, mla_bwd/mla_bwd.cu:1022-1025).  Calls queued
// on different streams get different scratch; a larger problem replaces the entry.
std::mutex g_ws_mutex;
std::map<std::pair<int, void*>, torch::Tensor> g_ws;

torch::Tensor workspace_for(size_t need, const torch::Device& dev, void* stream) {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    const std::pair<int, void*> key(dev.index(), stream);
    auto it = g_ws.find(key);
    if (it != g_ws.end() && static_cast<size_t>(it->second.numel()) >= need) return it->second;
    if (it != g_ws.end()) g_ws.erase(it);     // let the smaller one go first
    torch::Tensor buf = torch::empty({static_cast<int64_t>(need)}, torch::TensorOptions().dtype(torch::kUInt8).device(dev));
    buf.narrow(0, 0, 256).zero_();            // the device error word starts clear; the kernels only ever set it
    g_ws[key] = buf;
    return buf;
}

void check_input(const torch::Tensor& t, const char* name, const torch::Tensor& q, c10::ScalarType dtype) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.device() == q.device(), name, " must be on the same device as q");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
    TORCH_CHECK(t.scalar_type() == dtype, name, " has the wrong dtype");
}

std::tuple<torch::Tensor, torch::Tensor> mla_bwd(const torch::Tensor& q, const torch::Tensor& kv, const torch::Tensor& dO,
                                                 const torch::Tensor& lse, const torch::Tensor& O,
                                                 const torch::Tensor& indices, std::optional<double> sm_scale,
                                                 std::optional<int64_t> q_start_index_s, bool lse_is_base2) {
    // the reference's checks (mla_bwd/mla_bwd.cu:975-1015), widened to h_q = 8..128 and the 3-D kv / indices forms
    TORCH_CHECK(q.is_cuda(), "q must be a CUDA tensor");
    check_input(q, "q", q, torch::kBFloat16);
    check_input(kv, "kv", q, torch::kBFloat16);
    check_input(dO, "dO", q, torch::kBFloat16);
    check_input(O, "O", q, torch::kBFloat16);
    check_input(lse, "lse", q, torch::kFloat32);
    check_input(indices, "indices", q, torch::kInt32);
    TORCH_CHECK(q.dim() == 3 && q.size(2) == SMLA_D_QK, "q must have shape [s_q, h_q, 576]");
    TORCH_CHECK((kv.dim() == 2 || (kv.dim() == 3 && kv.size(1) == 1)) && kv.size(-1) == SMLA_D_QK,
                "kv must have shape [s_kv, 576] or [s_kv, 1, 576]");
    TORCH_CHECK(indices.dim() == 2 || (indices.dim() == 3 && indices.size(1) == 1),
                "indices must have shape [s_q, topk] or [s_q, 1, topk]");
    const int64_t s_q = q.size(0), h_q = q.size(1), s_kv = kv.size(0), topk = indices.size(-1);
    TORCH_CHECK(h_q > 0 && h_q <= 128 && h_q % 8 == 0, "h_q must be a multiple of 8 in [8, 128], got ", h_q);
    TORCH_CHECK(dO.dim() == 3 && dO.size(0) == s_q && dO.size(1) == h_q && dO.size(2) == SMLA_D_V, "dO must have shape [s_q, h_q, 512]");
    TORCH_CHECK(O.sizes() == dO.sizes(), "O must have shape [s_q, h_q, 512]");
    TORCH_CHECK(lse.dim() == 2 && lse.size(0) == s_q && lse.size(1) == h_q, "lse must have shape [s_q, h_q]");
    TORCH_CHECK(indices.size(0) == s_q, "indices first dim must equal s_q");
    TORCH_CHECK(topk > 0 && s_q > 0 && s_kv > 0, "s_q, s_kv and topk must be positive");

    const c10::cuda::CUDAGuard guard(q.device());
    torch::Tensor dQ = torch::empty_like(q);
    torch::Tensor dKV = torch::empty(kv.sizes(), q.options().dtype(torch::kFloat32));   // cleared by the library on the stream

    smla_bwd_params p{};
    p.q = q.data_ptr();
    p.kv = kv.data_ptr();
    p.dO = dO.data_ptr();
    p.lse = lse.data_ptr<float>();
    p.O = O.data_ptr();
    p.indices = indices.data_ptr<int32_t>();
    p.dQ = dQ.data_ptr();
    p.dKV = dKV.data_ptr<float>();
    p.s_q = static_cast<int32_t>(s_q);
    p.s_kv = static_cast<int32_t>(s_kv);
    p.h_q = static_cast<int32_t>(h_q);
    p.topk = static_cast<int32_t>(topk);
    p.sm_scale = sm_scale ? static_cast<float>(*sm_scale) : 0.0f;
    p.q_start_index_s = q_start_index_s ? static_cast<int32_t>(*q_start_index_s) : SMLA_NO_CAUSAL;
    p.lse_is_base2 = lse_is_base2 ? 1 : 0;
    p.query_meta = nullptr;

    const size_t need = smla_bwd_workspace_size(&p, 0);
    TORCH_CHECK(need > 0, "unsupported shapes for the sparse MLA backward");
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    torch::Tensor ws = workspace_for(need, q.device(), stream);
    const int st = smla_bwd_run(&p, ws.data_ptr(), static_cast<size_t>(ws.numel()), stream);
    TORCH_CHECK(st == SMLA_OK, "smla_bwd_run: ", smla_status_string(st), " (status ", st, ")");
    return {dQ, dKV};
}

// Synchronises the current stream of `device` and raises if a kernel of any call since the last check gave up on a wait.
void check_device_status(int64_t device) {
    const c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device)));
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    torch::Tensor ws;
    {
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        auto it = g_ws.find({static_cast<int>(device), stream});
        if (it == g_ws.end()) return;
        ws = it->second;
    }
    const int st = smla_bwd_status(ws.data_ptr(), stream);
    TORCH_CHECK(st == SMLA_OK, "sparse MLA backward: ", smla_status_string(st), " (device code ", smla_bwd_last_device_code(), ")");
}

void release_workspaces() {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    g_ws.clear();
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "Sparse MLA attention backward for sm_100a (drop-in for the reference's mla_bwd_cuda)";
    m.def("mla_bwd", &mla_bwd, py::arg("q"), py::arg("kv"), py::arg("dO"), py::arg("lse"), py::arg("O"), py::arg("indices"),
          py::arg("sm_scale") = py::none(), py::arg("q_start_index_s") = 0, py::arg("lse_is_base2") = true,
          "(dQ bf16 [s_q,h_q,576], dKV fp32 shaped like kv).  Defaults are the reference operator's: sm_scale 1/sqrt(576), "
          "base-2 lse, a slot counts only if idx <= query row (q_start_index_s = 0; None keeps only the range check).");
    m.def("check_device_status", &check_device_status, py::arg("device") = 0);
    m.def("release_workspaces", &release_workspaces);
}
