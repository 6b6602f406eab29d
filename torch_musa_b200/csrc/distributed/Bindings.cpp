// Python bindings of the distributed layer: process-group factory, backend-specific controls
// (flight recorder, fused-path switch, test hooks) and symmetric-memory views.
#include "distributed/ProcessGroupBCCL.h"
#include "distributed/SymmetricMemory.h"
#include "aten/Ops.h"
#include "core/Backend.h"

#include <ATen/Functions.h>

#include <pybind11/chrono.h>
#include <torch/csrc/utils/pybind.h>

namespace py = pybind11;

namespace b200 {

void init_distributed_bindings(py::module& m) {
  using dist::ProcessGroupBCCL;
  using dist::SymmetricMemory;

  // Layout of one sharded parameter group (kernels/fsdp_comm.cu): built once, passed to every launch.
  struct FsdpLayout { b200_fsdp_layout_t L{}; };
  py::class_<FsdpLayout, std::shared_ptr<FsdpLayout>>(m, "_FsdpLayout")
      .def(py::init([](std::vector<int64_t> shard_numel, std::vector<int64_t> shard_off, std::vector<int64_t> full_numel,
                       int64_t total) {
        TORCH_CHECK(!shard_numel.empty() && shard_numel.size() <= B200_FSDP_MAX_TENSORS, "fsdp layout: 1..",
                    B200_FSDP_MAX_TENSORS, " tensors per group");
        TORCH_CHECK(shard_off.size() == shard_numel.size() && full_numel.size() == shard_numel.size(), "fsdp layout: list lengths differ");
        auto l = std::make_shared<FsdpLayout>();
        l->L.n = (int)shard_numel.size();
        for (size_t i = 0; i < shard_numel.size(); ++i) {
          l->L.shard_numel[i] = shard_numel[i];
          l->L.shard_off[i] = shard_off[i];
          l->L.full_numel[i] = full_numel[i];
        }
        l->L.total = total;
        return l;
      }))
      .def_property_readonly("n", [](FsdpLayout& l) { return l.L.n; })
      .def_property_readonly("total", [](FsdpLayout& l) { return l.L.total; });
  m.attr("_FSDP_MAX_TENSORS") = (int)B200_FSDP_MAX_TENSORS;
  m.def("_comm_user_word0", [] { return b200_comm_user_word0(); });
  m.def("_comm_pad_words", [] { return b200_comm_pad_words(); });
  m.def("_comm_set_wait_ms", [](double ms) { b200_comm_set_wait_ms(ms); });
  m.def("_comm_get_wait_ms", [] { return b200_comm_get_wait_ms(); });

  py::class_<SymmetricMemory, std::shared_ptr<SymmetricMemory>>(m, "_SymmetricMemory")
      .def_property_readonly("ok", &SymmetricMemory::ok)
      .def_property_readonly("why_not", &SymmetricMemory::why_not)
      .def_property_readonly("rank", &SymmetricMemory::rank)
      .def_property_readonly("world", &SymmetricMemory::world)
      .def_property_readonly("half_bytes", &SymmetricMemory::half_bytes)
      .def("take_status", &SymmetricMemory::take_status)
      .def("local_tensor", [](SymmetricMemory& s, int64_t off, std::vector<int64_t> sizes, at::ScalarType dt) {
        return s.local_tensor(off, sizes, dt);
      })
      .def_property_readonly("size_bytes", [](SymmetricMemory& s) { return (int64_t)(2 * s.half_bytes()); })
      // ---- sharded-parameter collectives (kernels/fsdp_comm.cu); all on the device's current stream
      .def("fsdp_pack", [](SymmetricMemory& s, const std::shared_ptr<FsdpLayout>& lay, const std::vector<at::Tensor>& srcs,
                           int64_t shadow_off, at::ScalarType shadow_dtype, int64_t flag_word, int64_t version,
                           int64_t counter_word, int64_t n_ctas) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        TORCH_CHECK((int)srcs.size() == lay->L.n, "fsdp_pack: expected ", lay->L.n, " tensors");
        const void* ptrs[B200_FSDP_MAX_TENSORS];
        for (int i = 0; i < lay->L.n; ++i) {
          const at::Tensor& t = srcs[i];
          TORCH_CHECK(ops::on_device(t) && t.is_contiguous() && t.numel() >= lay->L.shard_numel[i] &&
                      t.scalar_type() == srcs[0].scalar_type() && t.device() == srcs[0].device(),
                      "fsdp_pack: tensor ", i, " must be a contiguous device shard of the group's dtype");
          ptrs[i] = t.const_data_ptr();
        }
        TORCH_CHECK(shadow_off >= 0 && shadow_off + lay->L.total * (int64_t)c10::elementSize(shadow_dtype) <=
                    (int64_t)(2 * s.half_bytes()), "fsdp_pack: the flat shard does not fit the arena");
        DeviceSwitch sw(srcs[0].device().index());
        cudaStream_t stream = ops::current_raw_stream(srcs[0]);
        ops::check_not_capturing(stream, "fsdp_pack");
        int e = b200_fsdp_pack(s.desc(), &lay->L, ptrs, ops::kdtype(srcs[0].scalar_type()), shadow_off,
                               ops::kdtype(shadow_dtype), (int)flag_word, (uint32_t)version, (int)counter_word,
                               (int)n_ctas, stream);
        TORCH_CHECK(e != (int)cudaErrorNotSupported, "fsdp_pack: dtype pair not covered");
        B200_KERNEL_CALL(e);
      })
      .def("fsdp_gather", [](SymmetricMemory& s, const std::shared_ptr<FsdpLayout>& lay, const std::vector<at::Tensor>& outs,
                             int64_t shadow_off, int64_t flag_word, int64_t version, int64_t n_ctas) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        TORCH_CHECK((int)outs.size() == lay->L.n, "fsdp_gather: expected ", lay->L.n, " tensors");
        void* ptrs[B200_FSDP_MAX_TENSORS];
        for (int i = 0; i < lay->L.n; ++i) {
          const at::Tensor& t = outs[i];
          TORCH_CHECK(ops::on_device(t) && t.is_contiguous() && t.numel() >= lay->L.shard_numel[i] * s.world() &&
                      t.scalar_type() == outs[0].scalar_type() && t.device() == outs[0].device(),
                      "fsdp_gather: output ", i, " must hold world * shard elements of the group's dtype");
          ptrs[i] = t.mutable_data_ptr();
        }
        DeviceSwitch sw(outs[0].device().index());
        cudaStream_t stream = ops::current_raw_stream(outs[0]);
        ops::check_not_capturing(stream, "fsdp_gather");
        B200_KERNEL_CALL(b200_fsdp_gather(s.desc(), &lay->L, ptrs, ops::kdtype(outs[0].scalar_type()), shadow_off,
                                          (int)flag_word, (uint32_t)version, (int)n_ctas, stream));
      })
      .def("fsdp_reduce", [](SymmetricMemory& s, const std::shared_ptr<FsdpLayout>& lay, const std::vector<at::Tensor>& grads,
                             int64_t stage_off, double scale, const std::optional<at::Tensor>& out32,
                             const std::vector<at::Tensor>& p32, const std::vector<at::Tensor>& m1,
                             const std::vector<at::Tensor>& m2, std::vector<double> hyper, int64_t shadow_off,
                             at::ScalarType shadow_dtype, int64_t shadow_word, int64_t shadow_version,
                             int64_t ready_word, int64_t ack_word, int64_t seq, int64_t ack_need, int64_t counter_word,
                             int64_t n_ctas) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        const int n = lay->L.n;
        TORCH_CHECK((int)grads.size() == n, "fsdp_reduce: expected ", n, " gradients");
        const void* gp[B200_FSDP_MAX_TENSORS];
        for (int i = 0; i < n; ++i) {
          const at::Tensor& t = grads[i];
          TORCH_CHECK(ops::on_device(t) && t.is_contiguous() && t.numel() == lay->L.full_numel[i] &&
                      t.scalar_type() == grads[0].scalar_type() && t.device() == grads[0].device(),
                      "fsdp_reduce: gradient ", i, " must be contiguous with the unsharded element count");
          gp[i] = t.const_data_ptr();
        }
        const int64_t esz = (int64_t)grads[0].element_size();
        TORCH_CHECK(stage_off >= 0 && (s.world() == 1 || stage_off + (int64_t)s.world() * lay->L.total * esz <=
                    (int64_t)(2 * s.half_bytes())), "fsdp_reduce: staging slots exceed the arena");
        b200_fsdp_adamw_t opt{};
        const bool fused_opt = !p32.empty();
        if (fused_opt) {
          TORCH_CHECK((int)p32.size() == n && (int)m1.size() == n && (int)m2.size() == n && hyper.size() == 6,
                      "fsdp_reduce: optimizer state lists must match the group");
          for (int i = 0; i < n; ++i) {
            for (const at::Tensor* t : {&p32[i], &m1[i], &m2[i]})
              TORCH_CHECK(ops::on_device(*t) && t->scalar_type() == at::kFloat && t->is_contiguous() &&
                          t->numel() >= lay->L.shard_numel[i] && t->device() == grads[0].device(),
                          "fsdp_reduce: master shards and moments must be fp32 with shard_numel elements");
            opt.p[i] = p32[i].data_ptr<float>();
            opt.m[i] = m1[i].data_ptr<float>();
            opt.v[i] = m2[i].data_ptr<float>();
          }
          opt.lr = (float)hyper[0]; opt.beta1 = (float)hyper[1]; opt.beta2 = (float)hyper[2]; opt.eps = (float)hyper[3];
          opt.weight_decay = (float)hyper[4]; opt.step = (float)hyper[5];
          opt.shadow_off = shadow_off;
          opt.shadow_dtype = ops::kdtype(shadow_dtype);
          opt.shadow_flag_word = (int)shadow_word;
          opt.shadow_version = (uint32_t)shadow_version;
          if (shadow_off >= 0)
            TORCH_CHECK(shadow_off + lay->L.total * (int64_t)c10::elementSize(shadow_dtype) <= (int64_t)(2 * s.half_bytes()),
                        "fsdp_reduce: the flat shard does not fit the arena");
        } else {
          TORCH_CHECK(out32 && ops::on_device(*out32) && out32->scalar_type() == at::kFloat && out32->is_contiguous() &&
                      out32->numel() >= lay->L.total, "fsdp_reduce: out32 must be an fp32 flat shard");
        }
        DeviceSwitch sw(grads[0].device().index());
        cudaStream_t stream = ops::current_raw_stream(grads[0]);
        ops::check_not_capturing(stream, "fsdp_reduce");
        int e = b200_fsdp_reduce(s.desc(), &lay->L, gp, ops::kdtype(grads[0].scalar_type()), stage_off, (float)scale,
                                 fused_opt ? nullptr : out32->data_ptr<float>(), fused_opt ? &opt : nullptr,
                                 (int)ready_word, (int)ack_word, (uint32_t)seq, (uint32_t)ack_need, (int)counter_word,
                                 (int)n_ctas, stream);
        TORCH_CHECK(e != (int)cudaErrorNotSupported, "fsdp_reduce: dtype combination not covered");
        B200_KERNEL_CALL(e);
      })
      // ---- expert-parallel token exchange (kernels/moe.cu); all on the device's current stream
      .def("moe_count", [](SymmetricMemory& s, const at::Tensor& idx, int64_t E) {
        TORCH_CHECK(ops::on_device(idx) && idx.scalar_type() == at::kInt && idx.is_contiguous(), "idx: int32 device tensor");
        DeviceSwitch sw(idx.device().index());
        at::Tensor slot = at::empty_like(idx);
        at::Tensor counts = at::empty({E}, idx.options());
        B200_KERNEL_CALL(b200_moe_count(idx.const_data_ptr<int>(), slot.data_ptr<int>(), counts.data_ptr<int>(),
                                        idx.numel(), (int)E, ops::current_raw_stream(idx)));
        return std::make_tuple(slot, counts);
      })
      .def("moe_dispatch", [](SymmetricMemory& s, const at::Tensor& x, const at::Tensor& idx, const at::Tensor& slot,
                              const at::Tensor& counts, int64_t E, int64_t cap_rows, int64_t recv_off,
                              int64_t counts_off) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        TORCH_CHECK(ops::on_device(x) && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(),
                    "moe_dispatch: x must be a contiguous bf16 [tokens, d] device tensor");
        TORCH_CHECK(idx.dim() == 2 && idx.size(0) == x.size(0) && idx.scalar_type() == at::kInt && idx.is_contiguous() &&
                    slot.sizes() == idx.sizes() && counts.numel() == E, "moe_dispatch: bad index tensors");
        const int T = (int)x.size(0), K = (int)idx.size(1), d = (int)x.size(1);
        TORCH_CHECK(recv_off >= 0 && recv_off + cap_rows * d * 2 <= (int64_t)(2 * s.half_bytes()) &&
                    counts_off + (int64_t)s.world() * E * 4 <= (int64_t)(2 * s.half_bytes()),
                    "moe_dispatch: receive buffer outside the arena");
        DeviceSwitch sw(x.device().index());
        at::Tensor pos = at::empty_like(idx);
        at::Tensor recv_counts = at::empty({E / s.world()}, idx.options());
        ops::check_not_capturing(ops::current_raw_stream(x), "moe_dispatch");
        const uint32_t epoch = s.next_epoch(nullptr);
        B200_KERNEL_CALL(b200_moe_dispatch(s.desc(), x.const_data_ptr(), idx.const_data_ptr<int>(),
                                           slot.const_data_ptr<int>(), counts.const_data_ptr<int>(), pos.data_ptr<int>(),
                                           recv_counts.data_ptr<int>(), T, K, d, (int)E, cap_rows, recv_off, counts_off,
                                           epoch, ops::current_raw_stream(x)));
        return std::make_tuple(pos, recv_counts);
      })
      .def("moe_gather", [](SymmetricMemory& s, const at::Tensor& idx, const at::Tensor& pos,
                            const std::optional<at::Tensor>& w, int64_t d, int64_t E, int64_t src_off) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        TORCH_CHECK(idx.dim() == 2 && idx.scalar_type() == at::kInt && pos.sizes() == idx.sizes() &&
                    pos.scalar_type() == at::kInt && idx.is_contiguous() && pos.is_contiguous(), "moe_gather: bad indices");
        TORCH_CHECK(!w || (w->scalar_type() == at::kFloat && w->sizes() == idx.sizes() && w->is_contiguous()),
                    "moe_gather: weights must be fp32 [tokens, k]");
        DeviceSwitch sw(idx.device().index());
        at::Tensor out = at::empty({idx.size(0), d}, idx.options().dtype(at::kBFloat16));
        ops::check_not_capturing(ops::current_raw_stream(idx), "moe_gather");
        const uint32_t epoch = s.next_epoch(nullptr);
        B200_KERNEL_CALL(b200_moe_gather(s.desc(), out.mutable_data_ptr(), idx.const_data_ptr<int>(),
                                         pos.const_data_ptr<int>(), w ? w->const_data_ptr<float>() : nullptr,
                                         (int)idx.size(0), (int)idx.size(1), (int)d, (int)E, src_off, epoch,
                                         ops::current_raw_stream(idx)));
        return out;
      })
      .def("moe_scatter", [](SymmetricMemory& s, const at::Tensor& x, const at::Tensor& idx, const at::Tensor& pos,
                             const std::optional<at::Tensor>& w, int64_t E, int64_t dst_off) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        TORCH_CHECK(ops::on_device(x) && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(),
                    "moe_scatter: x must be a contiguous bf16 [tokens, d] device tensor");
        TORCH_CHECK(idx.dim() == 2 && idx.size(0) == x.size(0) && pos.sizes() == idx.sizes(), "moe_scatter: bad indices");
        TORCH_CHECK(!w || (w->scalar_type() == at::kFloat && w->sizes() == idx.sizes() && w->is_contiguous()),
                    "moe_scatter: weights must be fp32 [tokens, k]");
        DeviceSwitch sw(x.device().index());
        ops::check_not_capturing(ops::current_raw_stream(x), "moe_scatter");
        const uint32_t epoch = s.next_epoch(nullptr);
        B200_KERNEL_CALL(b200_moe_scatter(s.desc(), x.const_data_ptr(), idx.const_data_ptr<int>(),
                                          pos.const_data_ptr<int>(), w ? w->const_data_ptr<float>() : nullptr,
                                          (int)x.size(0), (int)idx.size(1), (int)x.size(1), (int)E, dst_off, epoch,
                                          ops::current_raw_stream(x)));
      })
      // all-gather -> GEMM in one launch (kernels/gemm_tcgen05_2cta.cu): y = gather_rows(x_shard) @ w^T
      .def("gemm_allgather", [](SymmetricMemory& s, const at::Tensor& x_shard, const at::Tensor& w, int64_t shard_off,
                                at::Tensor& flags, int64_t copier_pairs) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        TORCH_CHECK(ops::on_device(x_shard) && x_shard.dim() == 2 && x_shard.is_contiguous() &&
                    (x_shard.scalar_type() == at::kBFloat16 || x_shard.scalar_type() == at::kHalf),
                    "gemm_allgather: x_shard must be a contiguous bf16/fp16 [rows, K] device tensor");
        TORCH_CHECK(ops::on_device(w) && w.dim() == 2 && w.scalar_type() == x_shard.scalar_type() &&
                    w.size(1) == x_shard.size(1) && w.device() == x_shard.device(), "gemm_allgather: w must be [N, K]");
        TORCH_CHECK(ops::on_device(flags) && flags.scalar_type() == at::kInt && flags.is_contiguous(),
                    "gemm_allgather: flags must be an int32 device tensor");
        const int64_t rows = x_shard.size(0), K = x_shard.size(1), N = w.size(0), M = rows * s.world();
        TORCH_CHECK(flags.numel() >= M / 256, "gemm_allgather: flags too short");
        const int64_t shard_bytes = rows * K * (int64_t)x_shard.element_size();
        TORCH_CHECK(shard_off >= 0 && shard_off + shard_bytes <= (int64_t)(2 * s.half_bytes()),
                    "gemm_allgather: shard does not fit the arena");
        DeviceSwitch sw(x_shard.device().index());
        s.local_tensor(shard_off, {rows, K}, x_shard.scalar_type()).copy_(x_shard);
        at::Tensor x_full = at::empty({M, K}, x_shard.options());
        at::Tensor y = at::empty({M, N}, x_shard.options());
        b200_gemm_desc_t g{};
        g.m = (int)M; g.n = (int)N; g.k = (int)K;
        g.a_kmajor = 1; g.lda = K;
        if (w.stride(1) == 1 && w.stride(0) >= K) { g.b_kmajor = 1; g.ldb = w.stride(0); }
        else if (w.stride(0) == 1 && w.stride(1) >= N) { g.b_kmajor = 0; g.ldb = w.stride(1); }
        else TORCH_CHECK(false, "gemm_allgather: w must be dense in one of its two dimensions");
        g.ldd = N;
        g.in_dtype = ops::kdtype(x_shard.scalar_type());
        g.out_dtype = g.in_dtype;
        g.batch = 1;
        g.alpha = 1.f;
        ops::check_not_capturing(ops::current_raw_stream(x_shard), "gemm_allgather");
        const uint32_t epoch = s.next_epoch(nullptr);
        int e = b200_gemm_allgather(&g, s.desc(), shard_off, x_full.mutable_data_ptr(),
                                    reinterpret_cast<uint32_t*>(flags.data_ptr<int>()), epoch, (int)copier_pairs,
                                    y.mutable_data_ptr(), w.const_data_ptr(), ops::current_raw_stream(x_shard));
        TORCH_CHECK(e != (int)cudaErrorNotSupported, "gemm_allgather: shape not covered (M % (256*world), K % 64, alignment)");
        B200_KERNEL_CALL(e);
        return std::make_tuple(y, x_full);
      })
      // GEMM -> reduce-scatter in one launch: y_shard = rows `rank` of sum_ranks(x_r @ w_r^T)
      .def("gemm_reduce_scatter", [](SymmetricMemory& s, const at::Tensor& x, const at::Tensor& w, int64_t partial_off,
                                     int64_t flag_off, int64_t reducer_pairs) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        TORCH_CHECK(ops::on_device(x) && x.dim() == 2 && x.is_contiguous() &&
                    (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf),
                    "gemm_reduce_scatter: x must be a contiguous bf16/fp16 [M, K] device tensor");
        TORCH_CHECK(ops::on_device(w) && w.dim() == 2 && w.scalar_type() == x.scalar_type() && w.size(1) == x.size(1) &&
                    w.device() == x.device(), "gemm_reduce_scatter: w must be [N, K]");
        const int64_t M = x.size(0), K = x.size(1), N = w.size(0), W = s.world();
        TORCH_CHECK(M % W == 0, "gemm_reduce_scatter: rows must divide by the world size");
        const int64_t flag_bytes = W * (M / 256 / W + 1) * (N / 256 + 1) * 2 * 4;
        TORCH_CHECK(partial_off >= 0 && partial_off + M * N * 2 <= (int64_t)(2 * s.half_bytes()) &&
                    flag_off + flag_bytes <= (int64_t)(2 * s.half_bytes()), "gemm_reduce_scatter: buffers exceed the arena");
        DeviceSwitch sw(x.device().index());
        at::Tensor y = at::empty({M / W, N}, x.options());
        b200_gemm_desc_t g{};
        g.m = (int)M; g.n = (int)N; g.k = (int)K;
        g.a_kmajor = 1; g.lda = K;
        if (w.stride(1) == 1 && w.stride(0) >= K) { g.b_kmajor = 1; g.ldb = w.stride(0); }
        else if (w.stride(0) == 1 && w.stride(1) >= N) { g.b_kmajor = 0; g.ldb = w.stride(1); }
        else TORCH_CHECK(false, "gemm_reduce_scatter: w must be dense in one of its two dimensions");
        g.ldd = N;
        g.in_dtype = ops::kdtype(x.scalar_type());
        g.out_dtype = g.in_dtype;
        g.batch = 1;
        g.alpha = 1.f;
        ops::check_not_capturing(ops::current_raw_stream(x), "gemm_reduce_scatter");
        const uint32_t epoch = s.next_epoch(nullptr);
        int e = b200_gemm_reduce_scatter(&g, s.desc(), partial_off, flag_off, epoch, (int)reducer_pairs,
                                         y.mutable_data_ptr(), x.const_data_ptr(), w.const_data_ptr(),
                                         ops::current_raw_stream(x));
        TORCH_CHECK(e != (int)cudaErrorNotSupported,
                    "gemm_reduce_scatter: shape not covered (M % (256*world), N % 256, K alignment, world <= 8)");
        B200_KERNEL_CALL(e);
        return y;
      })
      // reduce-scatter fused with the fp32 cast and the sharded AdamW step (kernels/comm.cu): grads [world * n]
      // (bf16 or fp32, one slice per rank) are summed over ranks for this rank's slice, scaled, and applied to the
      // owner's fp32 master shard / moments; p16 (optional) receives the updated bf16 shard.
      .def("reduce_scatter_adamw", [](SymmetricMemory& s, const at::Tensor& grads, at::Tensor& p32, at::Tensor& m,
                                      at::Tensor& v, const std::optional<at::Tensor>& p16, const at::Tensor& step,
                                      double lr, double beta1, double beta2, double eps, double wd, double scale) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        const int64_t n = p32.numel();
        TORCH_CHECK(ops::on_device(grads) && grads.is_contiguous() && grads.numel() == n * s.world() &&
                    (grads.scalar_type() == at::kBFloat16 || grads.scalar_type() == at::kFloat),
                    "reduce_scatter_adamw: grads must be contiguous bf16/fp32 with world * shard elements");
        for (const at::Tensor* t : {&p32, &m, &v})
          TORCH_CHECK(ops::on_device(*t) && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == n &&
                      t->device() == grads.device(), "reduce_scatter_adamw: p32 / m / v must be fp32 shards of equal size");
        TORCH_CHECK(!p16 || (ops::on_device(*p16) && p16->scalar_type() == at::kBFloat16 && p16->is_contiguous() &&
                             p16->numel() == n), "reduce_scatter_adamw: p16 must be a bf16 shard");
        TORCH_CHECK(ops::on_device(step) && step.scalar_type() == at::kFloat && step.numel() == 1, "step: fp32 scalar on the device");
        TORCH_CHECK(grads.numel() * (int64_t)grads.element_size() <= (int64_t)s.half_bytes(), "reduce_scatter_adamw: bucket exceeds the arena half");
        DeviceSwitch sw(grads.device().index());
        ops::check_not_capturing(ops::current_raw_stream(grads), "reduce_scatter_adamw");
        int64_t half = 0;
        const uint32_t epoch = s.next_epoch(&half);
        int e = b200_comm_reduce_scatter_adamw(s.desc(), ops::kdtype(grads.scalar_type()), grads.const_data_ptr(),
                                               p32.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                                               p16 ? p16->mutable_data_ptr() : nullptr, n, (float)scale, epoch, half,
                                               (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd,
                                               step.const_data_ptr<float>(), ops::current_raw_stream(grads));
        TORCH_CHECK(e != (int)cudaErrorNotSupported, "reduce_scatter_adamw: shard size must be a multiple of 8 and 16-byte aligned");
        B200_KERNEL_CALL(e);
      })
      .def("moe_gather_dot", [](SymmetricMemory& s, const at::Tensor& grad, const at::Tensor& idx, const at::Tensor& pos,
                                int64_t E, int64_t src_off) {
        TORCH_CHECK(s.ok(), "symmetric memory is not usable: ", s.why_not());
        TORCH_CHECK(ops::on_device(grad) && grad.scalar_type() == at::kBFloat16 && grad.dim() == 2 && grad.is_contiguous(),
                    "moe_gather_dot: grad must be a contiguous bf16 [tokens, d] device tensor");
        DeviceSwitch sw(grad.device().index());
        at::Tensor dw = at::empty(idx.sizes(), idx.options().dtype(at::kFloat));
        B200_KERNEL_CALL(b200_moe_gather_dot(s.desc(), grad.const_data_ptr(), idx.const_data_ptr<int>(),
                                             pos.const_data_ptr<int>(), dw.data_ptr<float>(), (int)grad.size(0),
                                             (int)idx.size(1), (int)grad.size(1), (int)E, src_off,
                                             ops::current_raw_stream(grad)));
        return dw;
      });

  // A stand-alone arena of `bytes` bytes mapped across the ranks that share `store` (world 1: no mapping).
  m.def("_create_symmetric_memory", [](c10::intrusive_ptr<c10d::Store> store, const std::string& key, int rank,
                                       int world, int device, int64_t bytes) {
    lazy_init();
    return std::make_shared<SymmetricMemory>(std::move(store), key, rank, world, (c10::DeviceIndex)device,
                                             (size_t)((bytes + 1) / 2 + 255) / 256 * 256);
  });

  m.def("_create_process_group", [](c10::intrusive_ptr<c10d::Store> store, int rank, int size,
                                    std::chrono::milliseconds timeout, py::object pg_options) {
    auto opts = c10::make_intrusive<ProcessGroupBCCL::Options>(true);
    opts->timeout = timeout;
    if (!pg_options.is_none()) {
      if (py::hasattr(pg_options, "is_high_priority_stream"))
        opts->is_high_priority_stream = pg_options.attr("is_high_priority_stream").cast<bool>();
      if (py::hasattr(pg_options, "use_fused_collectives"))
        opts->use_fused_collectives = pg_options.attr("use_fused_collectives").cast<bool>();
    }
    c10::intrusive_ptr<c10d::Backend> b = c10::make_intrusive<ProcessGroupBCCL>(std::move(store), rank, size, opts);
    return b;
  });

  auto cast = [](const c10::intrusive_ptr<c10d::Backend>& b) -> ProcessGroupBCCL* {
    auto* p = dynamic_cast<ProcessGroupBCCL*>(b.get());
    TORCH_CHECK(p, "expected a bccl backend object");
    return p;
  };
  m.def("_pg_dump_flight_recorder", [cast](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->dump_flight_recorder(); });
  m.def("_pg_fused_count", [cast](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->fused_collective_count(); });
  m.def("_pg_set_fused", [cast](const c10::intrusive_ptr<c10d::Backend>& b, bool on) { cast(b)->set_fused_collectives(on); });
  m.def("_pg_nccl_version", [cast](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->nccl_version(); });
  m.def("_pg_symmetric_memory", [cast](const c10::intrusive_ptr<c10d::Backend>& b, int device) {
    return cast(b)->symmetric_memory((c10::DeviceIndex)device);
  });
  m.def("_pg_make_test_work", [cast](const c10::intrusive_ptr<c10d::Backend>& b, std::chrono::milliseconds timeout) {
    return cast(b)->make_test_work(timeout);
  });
  m.def("_pg_error", [cast](const c10::intrusive_ptr<c10d::Backend>& b) { return (int)cast(b)->getError(); });
  m.def("_pg_comm_stream", [cast](const c10::intrusive_ptr<c10d::Backend>& b, int device) {
    auto s = cast(b)->comm_stream((c10::DeviceIndex)device).unwrap();
    return py::make_tuple((int64_t)s.id(), (int64_t)s.device_index(), (int64_t)s.device_type());
  });
  m.def("_nccl_version", [] {
    int v = 0;
    ncclGetVersion(&v);
    return v;
  });
}

}  // namespace b200
