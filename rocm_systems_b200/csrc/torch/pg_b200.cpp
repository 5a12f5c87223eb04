// torch.distributed backend "b200coll": a c10d::Backend whose collectives are the native
// library's (libb200coll.so). PyTorch is the framework layer; nothing here calls NCCL.
//
// Every collective is enqueued on a per-backend side stream that first waits for the caller's
// current stream; the returned Work holds a CUDA event, and Work::wait() makes the caller's
// stream wait for it without blocking the host (the semantics torch users have with NCCL).
// CPU tensors are not handled here: `rocm_systems_b200.parallel.init_process_group` registers
// the process group as "cpu:gloo,cuda:b200coll" so they go to gloo.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <pybind11/chrono.h>
#include <torch/extension.h>

#include <cstring>
#include <memory>
#include <mutex>

#include "b200coll/api_trace.h"
#include "b200coll/nccl.h"

namespace {

#define B200_TCHECK(call)                                                                         \
  do {                                                                                            \
    ncclResult_t r__ = (call);                                                                    \
    TORCH_CHECK(r__ == ncclSuccess, "b200coll: ", #call, " failed: ", ncclGetErrorString(r__), " — ", \
                ncclGetLastError(nullptr));                                                       \
  } while (0)

ncclDataType_t toNccl(at::ScalarType t) {
  switch (t) {
    case at::kChar: return ncclInt8;
    case at::kByte: return ncclUint8;
    case at::kBool: return ncclUint8;
    case at::kInt: return ncclInt32;
    case at::kLong: return ncclInt64;
    case at::kHalf: return ncclFloat16;
    case at::kFloat: return ncclFloat32;
    case at::kDouble: return ncclFloat64;
    case at::kBFloat16: return ncclBfloat16;
    case at::kFloat8_e4m3fn: return ncclFp8E4M3;
    case at::kFloat8_e5m2: return ncclFp8E5M2;
    case at::kUInt32: return ncclUint32;
    case at::kUInt64: return ncclUint64;
    default: TORCH_CHECK(false, "b200coll: unsupported dtype ", t);
  }
}

ncclRedOp_t toNccl(const c10d::ReduceOp& op, at::ScalarType t) {
  switch (op.op_) {
    case c10d::ReduceOp::SUM: return ncclSum;
    case c10d::ReduceOp::PRODUCT: return ncclProd;
    case c10d::ReduceOp::MIN: return ncclMin;
    case c10d::ReduceOp::MAX: return ncclMax;
    case c10d::ReduceOp::AVG: return ncclAvg;
    case c10d::ReduceOp::BOR: TORCH_CHECK(t == at::kBool, "b200coll: BOR only on bool tensors"); return ncclMax;
    case c10d::ReduceOp::BAND: TORCH_CHECK(t == at::kBool, "b200coll: BAND only on bool tensors"); return ncclMin;
    default: TORCH_CHECK(false, "b200coll: unsupported reduce op");
  }
}

class WorkB200 : public c10d::Work {
 public:
  WorkB200(c10d::OpType op, int rank, c10::Device dev) : c10d::Work(rank, op), dev_(dev) {}
  bool isCompleted() override { return event_.query(); }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds /*timeout*/ = kNoTimeout) override {
    // Stream-ordered: the caller's current stream waits for the collective.
    event_.block(c10::cuda::getCurrentCUDAStream(dev_.index()));
    if (blocking_) event_.synchronize();
    stash_.clear();
    return true;
  }
  void synchronize() override { wait(); }
  void blockCurrentStream() override { event_.block(c10::cuda::getCurrentCUDAStream(dev_.index())); }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
  std::vector<at::Tensor> result() override { return outputs_; }

  at::cuda::CUDAEvent event_{cudaEventDisableTiming};
  c10::Device dev_;
  std::vector<at::Tensor> stash_;    // keeps inputs/outputs alive until wait()
  std::vector<at::Tensor> outputs_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
  bool blocking_ = false;
};

class BackendB200 : public c10d::Backend {
 public:
  BackendB200(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout)
      : c10d::Backend(rank, size), store_(store), timeout_(timeout) {}

  ~BackendB200() override {
    try {
      shutdown();
    } catch (...) {
    }
  }

  const std::string getBackendName() const override { return "b200coll"; }
  bool supportsCoalescing() const override { return true; }

  void shutdown() override {
    std::lock_guard<std::mutex> lk(mu_);
    if (comm_) {
      c10::cuda::CUDAGuard g(dev_);
      cudaDeviceSynchronize();
      ncclCommDestroy(comm_);
      comm_ = nullptr;
    }
  }
  void abort() override {
    std::lock_guard<std::mutex> lk(mu_);
    if (comm_) {
      ncclCommAbort(comm_);
      comm_ = nullptr;
    }
  }
  c10d::ErrorType getError() override {
    if (!comm_) return c10d::ErrorType::SUCCESS;
    ncclResult_t e = ncclSuccess;
    ncclCommGetAsyncError(comm_, &e);
    if (e == ncclSuccess) return c10d::ErrorType::SUCCESS;
    return e == ncclRemoteError ? c10d::ErrorType::REMOTE_ERROR : c10d::ErrorType::COMM_ERROR;
  }
  void eagerConnectSingleDevice(at::Device device) override { ensure(device); }

  // ---- collectives ------------------------------------------------------------------------
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) override {
    TORCH_CHECK(tensors.size() == 1, "b200coll: one tensor per allreduce");
    auto& t = tensors[0];
    check(t);
    return run(c10d::OpType::ALLREDUCE, t.device(), {t}, {t}, [&](cudaStream_t s) {
      B200_TCHECK(ncclAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), toNccl(t.scalar_type()), toNccl(opts.reduceOp, t.scalar_type()), comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& opts) override {
    TORCH_CHECK(!tensors.empty(), "b200coll: empty tensor list");
    for (auto& t : tensors) check(t);
    return run(c10d::OpType::ALLREDUCE_COALESCED, tensors[0].device(), tensors, tensors, [&](cudaStream_t s) {
      for (auto& t : tensors)
        B200_TCHECK(ncclAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), toNccl(t.scalar_type()), toNccl(opts.reduceOp, t.scalar_type()), comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) override {
    TORCH_CHECK(tensors.size() == 1, "b200coll: one tensor per broadcast");
    auto& t = tensors[0];
    check(t);
    const int root = (int)opts.rootRank;
    return run(c10d::OpType::BROADCAST, t.device(), {t}, {t}, [&](cudaStream_t s) {
      B200_TCHECK(ncclBroadcast(t.data_ptr(), t.data_ptr(), t.numel(), toNccl(t.scalar_type()), root, comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) override {
    TORCH_CHECK(tensors.size() == 1, "b200coll: one tensor per reduce");
    auto& t = tensors[0];
    check(t);
    const int root = (int)opts.rootRank;
    return run(c10d::OpType::REDUCE, t.device(), {t}, {t}, [&](cudaStream_t s) {
      B200_TCHECK(ncclReduce(t.data_ptr(), t.data_ptr(), t.numel(), toNccl(t.scalar_type()), toNccl(opts.reduceOp, t.scalar_type()), root, comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& out, at::Tensor& in, const c10d::AllgatherOptions&) override {
    check(in);
    check(out);
    TORCH_CHECK(out.numel() == in.numel() * getSize(), "b200coll: all_gather_into_tensor output must be world_size x input");
    return run(c10d::OpType::_ALLGATHER_BASE, in.device(), {in}, {out}, [&](cudaStream_t s) {
      B200_TCHECK(ncclAllGather(in.data_ptr(), out.data_ptr(), in.numel(), toNccl(in.scalar_type()), comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins, const c10d::AllgatherOptions&) override {
    TORCH_CHECK(ins.size() == 1 && outs.size() == 1, "b200coll: one tensor per allgather");
    auto& in = ins[0];
    check(in);
    auto& list = outs[0];
    TORCH_CHECK((int)list.size() == getSize(), "b200coll: allgather output list must have world_size entries");
    at::Tensor flat = at::empty({getSize() * in.numel()}, in.options());
    return run(c10d::OpType::ALLGATHER, in.device(), {in, flat}, list, [&](cudaStream_t s) {
      B200_TCHECK(ncclAllGather(in.data_ptr(), flat.data_ptr(), in.numel(), toNccl(in.scalar_type()), comm_, s));
      c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(s, in.device().index()));
      for (int r = 0; r < getSize(); r++) list[r].copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(list[r]), true);
    });
  }

  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::AllgatherOptions&) override {
    TORCH_CHECK(outs.size() == ins.size() && !ins.empty(), "b200coll: mismatched coalesced all_gather lists");
    for (size_t i = 0; i < ins.size(); i++) { check(ins[i]); check(outs[i]); }
    std::vector<at::Tensor> keep = ins;
    return run(c10d::OpType::COALESCED, ins[0].device(), keep, outs, [&](cudaStream_t s) {
      for (size_t i = 0; i < ins.size(); i++)
        B200_TCHECK(ncclAllGather(ins[i].data_ptr(), outs[i].data_ptr(), ins[i].numel(), toNccl(ins[i].scalar_type()), comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& out, at::Tensor& in, const c10d::ReduceScatterOptions& opts) override {
    check(in);
    check(out);
    TORCH_CHECK(in.numel() == out.numel() * getSize(), "b200coll: reduce_scatter_tensor input must be world_size x output");
    return run(c10d::OpType::_REDUCE_SCATTER_BASE, in.device(), {in}, {out}, [&](cudaStream_t s) {
      B200_TCHECK(ncclReduceScatter(in.data_ptr(), out.data_ptr(), out.numel(), toNccl(in.scalar_type()), toNccl(opts.reduceOp, in.scalar_type()), comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins, const c10d::ReduceScatterOptions& opts) override {
    TORCH_CHECK(outs.size() == 1 && ins.size() == 1, "b200coll: one tensor per reduce_scatter");
    auto& out = outs[0];
    check(out);
    auto& list = ins[0];
    TORCH_CHECK((int)list.size() == getSize(), "b200coll: reduce_scatter input list must have world_size entries");
    at::Tensor flat = at::empty({getSize() * out.numel()}, out.options());
    std::vector<at::Tensor> keep = list;
    keep.push_back(flat);
    return run(c10d::OpType::REDUCE_SCATTER, out.device(), keep, {out}, [&](cudaStream_t s) {
      {
        c10::cuda::CUDAStreamGuard g(c10::cuda::getStreamFromExternal(s, out.device().index()));
        for (int r = 0; r < getSize(); r++) flat.narrow(0, r * out.numel(), out.numel()).copy_(list[r].reshape({-1}), true);
      }
      B200_TCHECK(ncclReduceScatter(flat.data_ptr(), out.data_ptr(), out.numel(), toNccl(out.scalar_type()), toNccl(opts.reduceOp, out.scalar_type()), comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::ReduceScatterOptions& opts) override {
    TORCH_CHECK(outs.size() == ins.size() && !ins.empty(), "b200coll: mismatched coalesced reduce_scatter lists");
    for (size_t i = 0; i < ins.size(); i++) { check(ins[i]); check(outs[i]); }
    std::vector<at::Tensor> keep = ins;
    return run(c10d::OpType::COALESCED, ins[0].device(), keep, outs, [&](cudaStream_t s) {
      for (size_t i = 0; i < ins.size(); i++)
        B200_TCHECK(ncclReduceScatter(ins[i].data_ptr(), outs[i].data_ptr(), outs[i].numel(), toNccl(ins[i].scalar_type()), toNccl(opts.reduceOp, ins[i].scalar_type()), comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& out, at::Tensor& in, std::vector<int64_t>& outSplit, std::vector<int64_t>& inSplit, const c10d::AllToAllOptions&) override {
    check(in);
    check(out);
    const int n = getSize();
    if (outSplit.empty() && inSplit.empty()) {
      TORCH_CHECK(in.numel() == out.numel() && in.numel() % n == 0, "b200coll: all_to_all_single needs equal, divisible sizes");
      return run(c10d::OpType::ALLTOALL_BASE, in.device(), {in}, {out}, [&](cudaStream_t s) {
        B200_TCHECK(ncclAllToAll(in.data_ptr(), out.data_ptr(), in.numel() / n, toNccl(in.scalar_type()), comm_, s));
      });
    }
    TORCH_CHECK((int)outSplit.size() == n && (int)inSplit.size() == n, "b200coll: split size lists must have world_size entries");
    const int64_t inRow = in.dim() ? in.numel() / std::max<int64_t>(in.size(0), 1) : 1;
    const int64_t outRow = out.dim() ? out.numel() / std::max<int64_t>(out.size(0), 1) : 1;
    std::vector<size_t> sc(n), sd(n), rc(n), rd(n);
    size_t so = 0, ro = 0;
    for (int i = 0; i < n; i++) {
      sc[i] = (size_t)(inSplit[i] * inRow);
      sd[i] = so;
      so += sc[i];
      rc[i] = (size_t)(outSplit[i] * outRow);
      rd[i] = ro;
      ro += rc[i];
    }
    return run(c10d::OpType::ALLTOALL_BASE, in.device(), {in}, {out}, [&, sc, sd, rc, rd](cudaStream_t s) {
      B200_TCHECK(ncclAllToAllv(in.data_ptr(), sc.data(), sd.data(), out.data_ptr(), rc.data(), rd.data(), toNccl(in.scalar_type()), comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::AllToAllOptions&) override {
    const int n = getSize();
    TORCH_CHECK((int)outs.size() == n && (int)ins.size() == n, "b200coll: all_to_all lists must have world_size entries");
    for (int i = 0; i < n; i++) { check(ins[i]); check(outs[i]); }
    std::vector<at::Tensor> keep = ins;
    return run(c10d::OpType::ALLTOALL, ins[0].device(), keep, outs, [&](cudaStream_t s) {
      B200_TCHECK(ncclGroupStart());
      for (int p = 0; p < n; p++) {
        B200_TCHECK(ncclSend(ins[p].data_ptr(), ins[p].numel(), toNccl(ins[p].scalar_type()), p, comm_, s));
        B200_TCHECK(ncclRecv(outs[p].data_ptr(), outs[p].numel(), toNccl(outs[p].scalar_type()), p, comm_, s));
      }
      B200_TCHECK(ncclGroupEnd());
    });
  }

  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int /*tag*/) override {
    TORCH_CHECK(tensors.size() == 1, "b200coll: one tensor per send");
    auto& t = tensors[0];
    check(t);
    return run(c10d::OpType::SEND, t.device(), {t}, {}, [&](cudaStream_t s) {
      B200_TCHECK(ncclSend(t.data_ptr(), t.numel(), toNccl(t.scalar_type()), dst, comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int /*tag*/) override {
    TORCH_CHECK(tensors.size() == 1, "b200coll: one tensor per recv");
    auto& t = tensors[0];
    check(t);
    return run(c10d::OpType::RECV, t.device(), {}, {t}, [&](cudaStream_t s) {
      B200_TCHECK(ncclRecv(t.data_ptr(), t.numel(), toNccl(t.scalar_type()), src, comm_, s));
    });
  }

  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins, const c10d::GatherOptions& opts) override {
    TORCH_CHECK(ins.size() == 1, "b200coll: one tensor per gather");
    auto& in = ins[0];
    check(in);
    const int root = (int)opts.rootRank, n = getSize();
    std::vector<at::Tensor> list;
    if (getRank() == root) {
      TORCH_CHECK(outs.size() == 1 && (int)outs[0].size() == n, "b200coll: gather output list must have world_size entries on the root");
      list = outs[0];
    }
    return run(c10d::OpType::GATHER, in.device(), {in}, list, [&, list](cudaStream_t s) {
      B200_TCHECK(ncclGroupStart());
      B200_TCHECK(ncclSend(in.data_ptr(), in.numel(), toNccl(in.scalar_type()), root, comm_, s));
      if (getRank() == root)
        for (int p = 0; p < n; p++) B200_TCHECK(ncclRecv(list[p].data_ptr(), list[p].numel(), toNccl(list[p].scalar_type()), p, comm_, s));
      B200_TCHECK(ncclGroupEnd());
    });
  }

  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins, const c10d::ScatterOptions& opts) override {
    TORCH_CHECK(outs.size() == 1, "b200coll: one tensor per scatter");
    auto& out = outs[0];
    check(out);
    const int root = (int)opts.rootRank, n = getSize();
    std::vector<at::Tensor> list;
    if (getRank() == root) {
      TORCH_CHECK(ins.size() == 1 && (int)ins[0].size() == n, "b200coll: scatter input list must have world_size entries on the root");
      list = ins[0];
    }
    return run(c10d::OpType::SCATTER, out.device(), list, {out}, [&, list](cudaStream_t s) {
      B200_TCHECK(ncclGroupStart());
      if (getRank() == root)
        for (int p = 0; p < n; p++) B200_TCHECK(ncclSend(list[p].data_ptr(), list[p].numel(), toNccl(list[p].scalar_type()), p, comm_, s));
      B200_TCHECK(ncclRecv(out.data_ptr(), out.numel(), toNccl(out.scalar_type()), root, comm_, s));
      B200_TCHECK(ncclGroupEnd());
    });
  }

  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts) override {
    c10::Device dev = dev_.is_cuda() && comm_ ? dev_ : c10::Device(c10::kCUDA, pickDevice(opts));
    auto w = run(c10d::OpType::BARRIER, dev, {}, {}, [&](cudaStream_t s) { B200_TCHECK(b200collBarrier(comm_, s)); });
    static_cast<WorkB200*>(w.get())->blocking_ = true;  // torch's barrier() blocks the host
    return w;
  }

  void startCoalescing() override {
    coalescing_++;
  }
  c10::intrusive_ptr<c10d::Work> endCoalescing() override {
    TORCH_CHECK(coalescing_ > 0, "b200coll: endCoalescing without startCoalescing");
    coalescing_--;
    if (!comm_) return nullptr;
    auto work = c10::make_intrusive<WorkB200>(c10d::OpType::COALESCED, getRank(), dev_);
    c10::cuda::CUDAGuard g(dev_);
    auto cs = commStream();
    work->event_.record(cs);
    work->stash_ = std::move(coalescedStash_);
    coalescedStash_.clear();
    makeFuture(*work, {}, cs);
    return work;
  }

 private:
  static void check(const at::Tensor& t) {
    TORCH_CHECK(t.is_cuda(), "b200coll: CUDA tensors only (CPU tensors belong to the gloo half of the process group)");
    TORCH_CHECK(t.is_contiguous(), "b200coll: tensors must be contiguous");
    TORCH_CHECK(!t.is_complex(), "b200coll: complex tensors are not supported");
  }

  int pickDevice(const c10d::BarrierOptions& opts) {
    if (!opts.device_ids.empty()) return (int)opts.device_ids[0];
    if (opts.device.has_value() && opts.device->is_cuda() && opts.device->has_index()) return opts.device->index();
    return c10::cuda::current_device();
  }

  void ensure(c10::Device dev) {
    std::lock_guard<std::mutex> lk(mu_);
    if (comm_) {
      TORCH_CHECK(dev == dev_, "b200coll: this process group is bound to ", dev_, ", got a tensor on ", dev);
      return;
    }
    TORCH_CHECK(dev.is_cuda(), "b200coll: needs a CUDA device");
    c10::cuda::CUDAGuard g(dev);
    ncclUniqueId id;
    const std::string key = "b200coll/uid/" + std::to_string(commCounter_);
    if (getRank() == 0) {
      B200_TCHECK(ncclGetUniqueId(&id));
      std::vector<uint8_t> v(sizeof(id));
      std::memcpy(v.data(), &id, sizeof(id));
      store_->set(key, v);
    } else {
      std::vector<uint8_t> v = store_->get(key);
      TORCH_CHECK(v.size() == sizeof(id), "b200coll: bad rendezvous id in the store");
      std::memcpy(&id, v.data(), sizeof(id));
    }
    B200_TCHECK(ncclCommInitRank(&comm_, getSize(), id, getRank()));
    dev_ = dev;
    stream_ = std::make_unique<c10::cuda::CUDAStream>(c10::cuda::getStreamFromPool(/*isHighPriority=*/true, dev.index()));
  }

  c10::cuda::CUDAStream commStream() { return *stream_; }

  void makeFuture(WorkB200& w, std::vector<at::Tensor> outs, c10::cuda::CUDAStream cs) {
    w.outputs_ = outs;
    w.future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), std::vector<c10::Device>{w.dev_});
    c10::cuda::CUDAStreamGuard sg(cs);  // the future records its event on the collective's stream
    w.future_->markCompleted(c10::IValue(outs));
  }

  template <typename F>
  c10::intrusive_ptr<c10d::Work> run(c10d::OpType op, c10::Device dev, std::vector<at::Tensor> ins, std::vector<at::Tensor> outs, F&& fn) {
    ensure(dev);
    c10::cuda::CUDAGuard g(dev);
    auto cur = c10::cuda::getCurrentCUDAStream(dev.index());
    auto cs = commStream();
    // The collective starts after everything already queued on the caller's stream.
    at::cuda::CUDAEvent ready(cudaEventDisableTiming);
    ready.record(cur);
    ready.block(cs);
    fn(cs.stream());
    auto work = c10::make_intrusive<WorkB200>(op, getRank(), dev);
    work->event_.record(cs);
    for (auto& t : ins) work->stash_.push_back(t);
    for (auto& t : outs) work->stash_.push_back(t);
    if (coalescing_ > 0)
      for (auto& t : work->stash_) coalescedStash_.push_back(t);
    makeFuture(*work, outs, cs);
    return work;
  }

  c10::intrusive_ptr<c10d::Store> store_;
  std::chrono::milliseconds timeout_;
  std::mutex mu_;
  ncclComm_t comm_ = nullptr;
  c10::Device dev_{c10::kCPU};
  std::unique_ptr<c10::cuda::CUDAStream> stream_;
  int coalescing_ = 0;
  std::vector<at::Tensor> coalescedStash_;
  int commCounter_ = 0;
};

c10::intrusive_ptr<c10d::Backend> createBackend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, const std::chrono::milliseconds& timeout) {
  return c10::make_intrusive<BackendB200>(store, rank, size, timeout);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "c10d backend of the b200coll collective library";
  m.def("create_backend", &createBackend, py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"));
  m.def("comm_handle", [](const c10::intrusive_ptr<c10d::Backend>& b) -> int64_t { return b->getID(); });
}
