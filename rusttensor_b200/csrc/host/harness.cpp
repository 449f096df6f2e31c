// librt_b200_host.so: the host side above the C ABI.
//
//  * `rth_*` engine API: the generic autograd engine (autograd.hpp) instantiated for the
//    CUDA backend, i.e. what a user of the reference gets from Tensor<B> / ops::* /
//    optim::* once B = B200Backend.
//  * `rth_dp_*`: the data-parallel training step built on top of it: forward + backward with the
//    all-reduce of the flat gradient buffer overlapped (the slice that is ready first goes out on a
//    side stream), one fused multi-tensor optimizer launch; forward, backward and the exchange are
//    replayed from a CUDA graph.
//
// No CPU fallback: every entry point fails with CudaError when no context exists.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unordered_map>

#include "b200_backend.hpp"
#include "engine_capi.hpp"

using rt::B200Backend;
using rt::Error;
using rt::ErrorKind;
using Tensor = rt::Tensor<B200Backend>;
using Storage = B200Backend::Storage;

RT_DEFINE_ENGINE_CAPI(rth, rt::B200Backend)

namespace {

// compiler-rt __powisf2 (f32::powi), for parity of Adam's bias correction on the host
// side when needed by callers.
struct DpTrainer {
  std::shared_ptr<rt::models::Trainer<B200Backend>> tr;
  int rank = 0, world = 1;
  std::vector<Storage> state1, state2;  // m / velocity, v
  Storage flat;                          // packed gradients (offsets padded to 4 elements)
  std::vector<int64_t> sizes, offsets;
  int64_t flat_len = 0;
  int64_t t = 0;
  // fixed device inputs + pinned host staging for the graph path
  std::vector<Tensor> inputs;
  std::vector<float*> pinned_in;
  float* pinned_loss = nullptr;
  Tensor captured_loss;
  rt_graph* graph = nullptr;    // forward + backward (up to the point where the early gradient slice is final)
  rt_graph* graph_b = nullptr;  // rest of the backward pass, when the capture was split there
  int early_lo = 0, early_hi = 0;  // parameters [early_lo, early_hi) are exchanged while graph_b runs
  bool packed_in_graph = false;    // the captured graph ends with the pack kernel
  // Device pointers the captured graph has baked in (inputs, parameters).  A copy-on-write of one of these tensors (a
  // view of an input or a parameter shares its buffer; make_unique then moves the tensor to a new buffer) would leave
  // the graph reading the old buffer, so every replay first compares and re-captures when one has moved.
  std::vector<const float*> captured_ptrs;
  bool have_loss = false;
  // exchange fused into the optimizer step over peer memory (rt_optimizer_step_multi_peers): two flat buffers that
  // alternate per step, a flag array written by the peers, and the peers' buffers as opened on this rank
  bool fused = false;
  Storage flat2[2], flag_store;
  std::vector<const float*> peer_flat[2];
  std::vector<int*> peer_flags;
  std::vector<void*> opened;
  // Step state on the device (RT_STEP_STATE_WORDS ints): exchange step, ready mark, optimizer step count.  With one
  // GPU and with the peer-memory exchange the optimizer step (and the exchange) is part of the captured graph and reads
  // its step numbers from here; the host's `t` is kept in step for checkpoints.
  Storage ctrl;
  int* ctrl_ptr() { return reinterpret_cast<int*>(ctrl.ptr()); }
  // RT_B200_DP_TRACE=1: time stamps (GPU nanosecond timer) around the parts of the captured step, read with rth_dp_trace
  rt::B200Backend::Storage trace;
  bool tracing = std::getenv("RT_B200_DP_TRACE") && std::getenv("RT_B200_DP_TRACE")[0] == '1';
  void stamp(int i) {
    if (!tracing) return;
    if (!trace.buf) trace = B200Backend::zeros(rt::Shape{32});
    B200Backend::check(rt_stamp(B200Backend::ctx(), reinterpret_cast<uint64_t*>(trace.ptr()) + i));
  }
  // RT_B200_DP_NCCL_GRAPH=1: the NCCL all-reduce and the optimizer are recorded in the step's graph too (pack -> all-reduce ->
  // optimizer with the step count on the device), one launch per step like the single-GPU and the peer-memory steps.
  bool nccl_in_graph = std::getenv("RT_B200_DP_NCCL_GRAPH") && std::getenv("RT_B200_DP_NCCL_GRAPH")[0] == '1';
  bool update_in_stream() const { return tr->w.optimizer != 0 && (world == 1 || fused || (nccl_in_graph && !overlap_exchange)); }
  // pipelined steps: double-buffered uploads, two loss slots with completion events
  std::vector<rt_upload*> uploads;
  float* pipe_loss[2] = {nullptr, nullptr};
  rt_event* pipe_done[2] = {nullptr, nullptr};
  int64_t pipe_steps = 0;
  // device-resident data set (data::get_random_batch without the host round trip): per step only the row numbers
  // travel; the rows are gathered on the device straight into the step's input tensors
  std::vector<Storage> dataset;          // one [rows, sample elements] tensor per input
  int64_t dataset_rows = 0;
  rt_upload* idx_upload = nullptr;  // row numbers of the next batch: pinned buffers, copy stream and staging like any input
  Storage idx_dev;
  // RT_B200_DP_OVERLAP=1 sends the early gradient slice while the backward pass is still running.  Off by default:
  // with this model (1.7 MB of gradients) on two B200s the extra NCCL launch and graph launch cost more than the
  // overlap hides (0.371 ms per step against 0.362 ms).
  bool overlap_exchange = std::getenv("RT_B200_DP_OVERLAP") && std::getenv("RT_B200_DP_OVERLAP")[0] == '1';

  ~DpTrainer() {
    rt_ctx* c = B200Backend::ctx_slot();
    if (!c) return;
    for (void* p : opened) rt_ipc_close(c, p);
    for (rt_upload* u : uploads) rt_upload_destroy(c, u);
    for (int i = 0; i < 2; ++i) {
      if (pipe_loss[i]) rt_host_free(c, pipe_loss[i]);
      if (pipe_done[i]) rt_event_destroy(c, pipe_done[i]);
    }
    if (idx_upload) rt_upload_destroy(c, idx_upload);
    if (graph) rt_graph_destroy(c, graph);
    if (graph_b) rt_graph_destroy(c, graph_b);
    for (float* p : pinned_in) rt_host_free(c, p);
    if (pinned_loss) rt_host_free(c, pinned_loss);
  }

  void setup() {
    auto& w = tr->w;
    int64_t off = 0;
    for (auto& p : w.params) {
      int64_t n = (int64_t)p.size();
      sizes.push_back(n);
      offsets.push_back(off);
      off += (n + 3) & ~int64_t(3);
      if (w.optimizer != 0) state1.push_back(B200Backend::zeros(p.shape()));
      if (w.optimizer == 1) state2.push_back(B200Backend::zeros(p.shape()));
    }
    flat_len = off;
    ctrl = B200Backend::zeros(rt::Shape{RT_STEP_STATE_WORDS});  // all-zero bits: step 0, nothing ready, t = 0
    if (world > 1) flat = B200Backend::zeros(rt::Shape{(size_t)flat_len});
    for (auto& s : w.input_shapes) {
      // C4's first input receives a gradient ("backward to input")
      bool rg = (w.config == rt::models::C4_CONV_CONVT) && inputs.empty();
      inputs.push_back(Tensor::zeros(s, rg));
      void* hp = nullptr;
      B200Backend::check(rt_host_alloc(B200Backend::ctx(), sizeof(float) * rt::shape_numel(s), &hp));
      pinned_in.push_back((float*)hp);
    }
    void* lp = nullptr;
    B200Backend::check(rt_host_alloc(B200Backend::ctx(), sizeof(float), &lp));
    pinned_loss = (float*)lp;
  }

  // Packs the gradients of parameters [lo, hi) into their slice of the flat buffer and all-reduces that slice.
  void pack_and_reduce(int lo, int hi, bool do_pack = true, bool do_reduce = true) {
    if (lo >= hi) return;
    auto& w = tr->w;
    std::vector<const float*> srcs;
    for (int i = lo; i < hi; ++i) {
      auto& p = w.params[i];
      if (!p.grad()) throw Error(ErrorKind::NoGradientError, "parameter received no gradient");
      srcs.push_back(p.grad()->ptr());
    }
    rt_ctx* c = B200Backend::ctx();
    const int64_t begin = offsets[lo], end = hi < (int)offsets.size() ? offsets[hi] : flat_len;
    float* dst = flat.ptr();
    if (do_pack)
      B200Backend::check(rt_pack_flat(c, hi - lo, srcs.data(), sizes.data() + lo, dst + begin, w.clip_grads ? 1 : 0, w.clip_lo,
                                      w.clip_hi));
    if (do_reduce) B200Backend::check(rt_dp_allreduce_sum(c, dst + begin, end - begin));
  }

  // forward + backward (+ gradient exchange when world > 1); everything asynchronous.
  // Data parallel: as soon as the backward walk has finalised at least half of the gradient elements (for a CNN the
  // fully connected layers, reached first), the largest contiguous run of ready parameters becomes the early slice,
  // which is packed and all-reduced on a side stream while the rest of the backward pass runs; the remaining slices
  // follow on the main stream.  NCCL stays outside CUDA graphs (a captured all-reduce measured ~40 us slower per
  // step than an eager one): under capture the graph is split at that point instead, and the caller runs the
  // exchange between the two replays (exchange_early / exchange_rest).
  Tensor forward_backward(bool capturing) {
    auto& w = tr->w;
    rt_ctx* cx = B200Backend::ctx();
    if (update_in_stream()) {
      own_buffers();  // the launches below (and the graph, when capturing) keep these pointers
      stamp(0);
      B200Backend::check(rt_dp_step_begin(cx, ctrl_ptr()));
    }
    for (auto& p : w.params) p.zero_grad();
    for (auto& x : inputs) x.zero_grad();
    Tensor loss = rt::models::forward_loss(w, inputs);
    early_lo = early_hi = 0;
    if (update_in_stream() || world == 1 || fused) {
      stamp(1);
      loss.backward();
      stamp(2);
      if (update_in_stream()) update_on_device();
      stamp(6);
      return loss;
    }
    const int n = (int)w.params.size();
    std::unordered_map<size_t, int> index;
    for (int i = 0; i < n; ++i) index[w.params[i].id()] = i;
    std::vector<char> ready(n, 0);
    int64_t ready_elems = 0, total = 0;
    for (int i = 0; i < n; ++i) total += sizes[i];
    bool fired = false;
    rt_ctx* c = B200Backend::ctx();
    struct HookGuard {
      ~HookGuard() { Tensor::leaf_ready_hook() = nullptr; }
    } guard;
    Tensor::leaf_ready_hook() = [&](const Tensor& leaf) {
      auto it = index.find(leaf.id());
      if (it == index.end() || ready[it->second]) return;
      ready[it->second] = 1;
      ready_elems += sizes[it->second];
      if (fired || ready_elems * 2 < total || ready_elems == total || !overlap_exchange || fused) return;
      int64_t best = 0;
      for (int i = 0; i < n;) {  // largest contiguous run of ready parameters
        if (!ready[i]) { ++i; continue; }
        int j = i;
        int64_t run = 0;
        while (j < n && ready[j]) run += sizes[j++];
        if (run > best) { best = run; early_lo = i; early_hi = j; }
        i = j;
      }
      fired = true;
      if (capturing) {  // split the capture here; the exchange of the early slice runs between the two replays
        B200Backend::check(rt_graph_end(c, &graph));
        B200Backend::check(rt_graph_begin(c));
      } else {
        exchange_early();
      }
    };
    loss.backward();
    Tensor::leaf_ready_hook() = nullptr;
    if (!capturing) exchange_rest();
    else if (!fused && !fired) {  // single exchange: the pack kernel is recorded with the backward pass
      pack_and_reduce(0, n, true, false);
      packed_in_graph = true;
    }
    return loss;
  }
  void exchange_early() {
    if (world == 1 || early_lo >= early_hi) return;
    rt_ctx* c = B200Backend::ctx();
    B200Backend::check(rt_side_stream_begin(c));
    try {
      pack_and_reduce(early_lo, early_hi);
    } catch (...) {
      rt_side_stream_end(c);
      throw;
    }
    B200Backend::check(rt_side_stream_end(c));
  }
  void exchange_rest() {
    if (world == 1 || fused) return;  // fused: pack, signal, wait and update are part of forward_backward's stream work
    if (packed_in_graph && graph) {  // replaying: the graph has already packed
      pack_and_reduce(0, (int)tr->w.params.size(), false, true);
      return;
    }
    pack_and_reduce(0, early_lo);
    pack_and_reduce(early_hi, (int)tr->w.params.size());
    B200Backend::check(rt_side_stream_join(B200Backend::ctx()));
  }

  // Peer-memory exchange, set-up part 1: allocate the buffers the peers will read / write and export their handles
  // (3 x RT_IPC_HANDLE_BYTES: flat buffer 0, flat buffer 1, flag array).
  void fused_export(uint8_t* out) {
    if (world == 1) throw Error::invalid_op("fused exchange needs more than one rank");
    if (graph) throw Error::invalid_op("set up the fused exchange before the first captured step");
    rt_ctx* c = B200Backend::ctx();
    // Exported blocks are at least 2 MiB: the driver may carve smaller cudaMalloc requests out of a shared block, and an
    // IPC handle always maps the whole underlying block from its start.
    const size_t min_elems = (size_t)1 << 19;
    for (int i = 0; i < 2; ++i) {
      flat2[i] = B200Backend::zeros(rt::Shape{std::max((size_t)flat_len, min_elems)});
      B200Backend::check(rt_ipc_export(c, flat2[i].ptr(), out + i * RT_IPC_HANDLE_BYTES));
    }
    flag_store = B200Backend::zeros(rt::Shape{min_elems});  // all-zero bits = step 0; slot r is written by rank r
    B200Backend::check(rt_ipc_export(c, flag_store.ptr(), out + 2 * RT_IPC_HANDLE_BYTES));
    B200Backend::check(rt_sync(c));
  }
  // Part 2: `all` holds every rank's three handles in rank order.
  void fused_connect(const uint8_t* all) {
    if (!flat2[0].buf) throw Error::invalid_op("fused_export must run first");
    rt_ctx* c = B200Backend::ctx();
    for (int i = 0; i < 2; ++i) peer_flat[i].assign(world, nullptr);
    peer_flags.assign(world, nullptr);
    for (int r = 0; r < world; ++r) {
      if (r == rank) {
        peer_flat[0][r] = flat2[0].ptr();
        peer_flat[1][r] = flat2[1].ptr();
        peer_flags[r] = reinterpret_cast<int*>(flag_store.ptr());
        continue;
      }
      void* p[3] = {nullptr, nullptr, nullptr};
      for (int i = 0; i < 3; ++i) {
        B200Backend::check(rt_ipc_open(c, all + ((size_t)r * 3 + i) * RT_IPC_HANDLE_BYTES, &p[i]));
        opened.push_back(p[i]);
      }
      peer_flat[0][r] = static_cast<const float*>(p[0]);
      peer_flat[1][r] = static_cast<const float*>(p[1]);
      peer_flags[r] = static_cast<int*>(p[2]);
    }
    fused = true;
  }

  // Parameters and optimizer state get buffers of their own (copy on write) before their pointers go into launches.
  void own_buffers() {
    auto& w = tr->w;
    for (size_t i = 0; i < w.params.size(); ++i) {
      B200Backend::make_unique(w.params[i].data_mut());
      if (w.optimizer != 0) B200Backend::make_unique(state1[i]);
      if (w.optimizer == 1) B200Backend::make_unique(state2[i]);
    }
  }
  struct UpdatePointers {
    std::vector<float*> ps, s1, s2;
    std::vector<const float*> gs;
  };
  UpdatePointers update_pointers(const float* flat_base) {
    auto& w = tr->w;
    UpdatePointers u;
    for (size_t i = 0; i < w.params.size(); ++i) {
      auto& p = w.params[i];
      u.ps.push_back(p.data().ptr());
      u.s1.push_back(state1[i].ptr());
      u.s2.push_back(w.optimizer == 1 ? state2[i].ptr() : nullptr);
      if (flat_base) u.gs.push_back(flat_base + offsets[i]);
      else {
        if (!p.grad()) throw Error(ErrorKind::NoGradientError, "parameter received no gradient");
        u.gs.push_back(p.grad()->ptr());
      }
    }
    return u;
  }
  // The optimizer step as stream work behind the backward pass, with every step number read on the device: one GPU
  // (fused multi-tensor launch) or the peer-memory exchange (pack into this step's flat buffer, tell the peers, wait for
  // theirs, then read all ranks' gradients inside the optimizer kernel).  Capturable.
  void update_on_device() {
    auto& w = tr->w;
    rt_ctx* c = B200Backend::ctx();
    const int kind = w.optimizer == 1 ? 1 : 2;
    if (!fused && world > 1) {  // NCCL inside the step: pack (with the clip), all-reduce, optimizer on the summed buffer
      pack_and_reduce(0, (int)w.params.size(), true, true);
      UpdatePointers u = update_pointers(flat.ptr());
      B200Backend::check(rt_optimizer_step_multi_device_t(c, kind, (int)u.ps.size(), u.ps.data(), u.gs.data(), u.s1.data(), u.s2.data(),
                                                          sizes.data(), w.lr, w.beta1, w.beta2, w.eps, w.momentum, ctrl_ptr(),
                                                          1.0f / (float)world, 0, w.clip_lo, w.clip_hi));
      return;
    }
    if (!fused) {
      UpdatePointers u = update_pointers(nullptr);
      B200Backend::check(rt_optimizer_step_multi_device_t(c, kind, (int)u.ps.size(), u.ps.data(), u.gs.data(), u.s1.data(), u.s2.data(),
                                                          sizes.data(), w.lr, w.beta1, w.beta2, w.eps, w.momentum, ctrl_ptr(), 1.0f,
                                                          w.clip_grads ? 1 : 0, w.clip_lo, w.clip_hi));
      return;
    }
    std::vector<const float*> srcs;
    for (auto& p : w.params) {
      if (!p.grad()) throw Error(ErrorKind::NoGradientError, "parameter received no gradient");
      srcs.push_back(p.grad()->ptr());
    }
    // pack (its last block signals the peers) -> wait -> optimizer, all on one stream: a kernel that waits for a peer never
    // runs beside work of this rank that the peer in turn waits for (two streams may share a hardware queue, and the pack
    // could then sit behind the spinning wait).
    B200Backend::check(rt_pack_flat_signal(c, (int)srcs.size(), srcs.data(), sizes.data(), flat2[0].ptr(), flat2[1].ptr(), ctrl_ptr(),
                                           w.clip_grads ? 1 : 0, w.clip_lo, w.clip_hi, peer_flags.data(), rank, world));
    stamp(3);
    B200Backend::check(rt_dp_wait_peers(c, reinterpret_cast<const int*>(flag_store.ptr()), rank, world, ctrl_ptr(), 0));
    stamp(4);
    UpdatePointers u = update_pointers(flat2[0].ptr());
    B200Backend::check(rt_optimizer_step_multi_peers(c, kind, (int)u.ps.size(), u.ps.data(), u.gs.data(), u.s1.data(), u.s2.data(),
                                                     sizes.data(), w.lr, w.beta1, w.beta2, w.eps, w.momentum, 1.0f / (float)world,
                                                     peer_flat[0].data(), peer_flat[1].data(), rank, world, ctrl_ptr()));
  }

  // After the backward pass (and the exchange): the optimizer step, unless it already is part of the stream work of
  // forward_backward.  The host's step count moves either way.
  void exchange_and_update() {
    auto& w = tr->w;
    rt_ctx* c = B200Backend::ctx();
    if (w.optimizer == 0) return;
    t += 1;
    if (update_in_stream()) return;
    own_buffers();
    UpdatePointers u = update_pointers(flat.ptr());
    // the clip already happened while packing
    B200Backend::check(rt_optimizer_step_multi(c, w.optimizer == 1 ? 1 : 2, (int)u.ps.size(), u.ps.data(), u.gs.data(), u.s1.data(),
                                               u.s2.data(), sizes.data(), w.lr, w.beta1, w.beta2, w.eps, w.momentum, t,
                                               1.0f / (float)world, 0, w.clip_lo, w.clip_hi));
  }
  // Restores the optimizer's step count (checkpoints): host and device copies.
  void set_step(int64_t v) {
    t = v;
    const int tv = (int)v;
    B200Backend::check(rt_memcpy_h2d(B200Backend::ctx(), ctrl_ptr() + 2, &tv, sizeof(int)));
  }

  void upload_inputs(const float* const* host_inputs, int n, bool from_pinned) {
    rt_ctx* c = B200Backend::ctx();
    if (n != (int)inputs.size()) throw Error::invalid_op("wrong number of inputs");
    for (int i = 0; i < n; ++i) {
      size_t bytes = sizeof(float) * inputs[i].size();
      B200Backend::make_unique(inputs[i].data_mut());
      if (from_pinned) B200Backend::check(rt_memcpy_h2d_async(c, inputs[i].data().ptr(), host_inputs[i], bytes));
      else {
        std::memcpy(pinned_in[i], host_inputs[i], bytes);
        B200Backend::check(rt_memcpy_h2d_async(c, inputs[i].data().ptr(), pinned_in[i], bytes));
      }
    }
  }

  // One eager step (host builds the graph of tensors every time).
  float step_eager(const float* const* host_inputs, int n) {
    if (graph) throw Error::invalid_op("step_eager after capture: use step_graph");
    upload_inputs(host_inputs, n, false);
    captured_loss = forward_backward(false);
    have_loss = true;
    exchange_and_update();
    rt_ctx* c = B200Backend::ctx();
    B200Backend::check(rt_memcpy_d2h_async(c, pinned_loss, captured_loss.data().ptr(), sizeof(float)));
    B200Backend::check(rt_sync(c));
    return *pinned_loss;
  }

  // Records forward+backward(+pack) once; afterwards a step is: H2D of the inputs,
  // one graph launch, the all-reduce, one optimizer launch, D2H of the loss.
  void capture() {
    rt_ctx* c = B200Backend::ctx();
    if (graph) return;
    captured_loss = Tensor();
    have_loss = false;
    B200Backend::check(rt_graph_begin(c));
    rt_graph* last = nullptr;
    try {
      captured_loss = forward_backward(true);
    } catch (...) {
      rt_graph* g = nullptr;
      rt_graph_end(c, &g);
      if (g) rt_graph_destroy(c, g);
      if (graph) {
        rt_graph_destroy(c, graph);
        graph = nullptr;
      }
      throw;
    }
    B200Backend::check(rt_graph_end(c, &last));
    if (graph) graph_b = last;  // the hook closed the first part
    else graph = last;
    have_loss = true;
    captured_ptrs = graph_pointers();
  }

  std::vector<const float*> graph_pointers() {
    std::vector<const float*> v;
    for (auto& x : inputs) v.push_back(x.data().ptr());
    for (auto& p : tr->w.params) v.push_back(p.data().ptr());
    if (update_in_stream()) {  // the captured optimizer launch holds the state pointers too
      for (auto& st : state1) v.push_back(st.ptr());
      for (auto& st : state2) v.push_back(st.ptr());
    }
    return v;
  }
  // A parameter or state buffer that somebody else holds too (a tensor handle obtained between steps) must not be
  // updated in place by the captured optimizer launch: such buffers are replaced by copies, which moves their pointers.
  bool shared_update_buffers() {
    if (!update_in_stream()) return false;
    for (auto& p : tr->w.params)
      if (p.data().buf && p.data().buf.use_count() > 1) return true;
    for (auto& st : state1)
      if (st.buf && st.buf.use_count() > 1) return true;
    for (auto& st : state2)
      if (st.buf && st.buf.use_count() > 1) return true;
    return false;
  }
  void invalidate_capture() {
    if (!graph) return;
    rt_ctx* c = B200Backend::ctx();
    B200Backend::check(rt_sync(c));
    rt_graph_destroy(c, graph);
    graph = nullptr;
    if (graph_b) {
      rt_graph_destroy(c, graph_b);
      graph_b = nullptr;
    }
    packed_in_graph = false;
  }
  void ensure_capture_is_current() {
    if (!graph) return;
    if (shared_update_buffers()) own_buffers();
    if (captured_ptrs == graph_pointers()) return;
    rt_ctx* c = B200Backend::ctx();
    B200Backend::check(rt_sync(c));  // nothing of the stale graph may still be running
    rt_graph_destroy(c, graph);
    graph = nullptr;
    if (graph_b) {
      rt_graph_destroy(c, graph_b);
      graph_b = nullptr;
    }
    packed_in_graph = false;
    capture();
  }

  // One replay of the captured step, with the gradient exchange between / after the two parts.
  void replay() {
    ensure_capture_is_current();
    rt_ctx* c = B200Backend::ctx();
    B200Backend::check(rt_graph_launch(c, graph));
    if (graph_b) {
      exchange_early();  // side stream: overlaps graph_b
      B200Backend::check(rt_graph_launch(c, graph_b));
    }
    exchange_rest();
  }

  // host_inputs == nullptr: reuse the inputs already resident on the device
  void step_graph_async(const float* const* host_inputs, int n, bool from_pinned) {
    if (!graph) capture();
    rt_ctx* c = B200Backend::ctx();
    if (host_inputs) upload_inputs(host_inputs, n, from_pinned);
    replay();
    exchange_and_update();
    if (host_inputs) B200Backend::check(rt_memcpy_d2h_async(c, pinned_loss, captured_loss.data().ptr(), sizeof(float)));
  }

  // ---- pipelined steps: the host runs one step ahead of the device ----
  void pipe_setup() {
    if (!uploads.empty()) return;
    rt_ctx* c = B200Backend::ctx();
    for (auto& x : inputs) {
      rt_upload* u = nullptr;
      B200Backend::check(rt_upload_create(c, sizeof(float) * x.size(), &u));
      uploads.push_back(u);
    }
    for (int i = 0; i < 2; ++i) {
      void* lp = nullptr;
      B200Backend::check(rt_host_alloc(c, sizeof(float), &lp));
      pipe_loss[i] = (float*)lp;
      B200Backend::check(rt_event_create(c, &pipe_done[i]));
    }
  }
  float* pipe_buffer(int i) {
    pipe_setup();
    void* p = nullptr;
    B200Backend::check(rt_upload_host_buffer(B200Backend::ctx(), uploads.at(i), &p));
    return (float*)p;
  }
  // Submits the buffers handed out by pipe_buffer, enqueues the step and the read-back of its loss, and
  // returns the loss of the PREVIOUS pipelined step (its work finished while this one was being enqueued).
  bool step_pipelined(float* prev_loss) {
    pipe_setup();
    if (!graph) capture();
    rt_ctx* c = B200Backend::ctx();
    // all inputs in one staging -> tensor kernel (one call per 8 inputs), the loss by a store to pinned memory: no copy-engine
    // round trip sits between two replays of the step
    std::vector<void*> dsts;
    for (auto& x : inputs) {
      B200Backend::make_unique(x.data_mut());
      dsts.push_back(x.data().ptr());
    }
    for (size_t i = 0; i < inputs.size(); i += 8)
      B200Backend::check(rt_upload_submit_all(c, uploads.data() + i, dsts.data() + i, (int)std::min<size_t>(8, inputs.size() - i)));
    replay();
    exchange_and_update();
    const int k = (int)(pipe_steps & 1);
    B200Backend::check(rt_publish_to_host(c, pipe_loss[k], captured_loss.data().ptr(), 1));
    B200Backend::check(rt_event_record(c, pipe_done[k]));
    const bool have_prev = pipe_steps > 0;
    if (have_prev) {
      B200Backend::check(rt_dp_wait_event(c, pipe_done[k ^ 1]));
      *prev_loss = *pipe_loss[k ^ 1];
    }
    ++pipe_steps;
    return have_prev;
  }
  // ---- steps fed from a data set that lives on the device ----
  void attach_dataset(const float* const* host_arrays, int n_arrays, int64_t rows) {
    if (n_arrays != (int)inputs.size()) throw Error::invalid_op("attach_dataset: one array per input");
    if (rows <= 0 || rows >= (1ll << 31)) throw Error::invalid_op("attach_dataset: row count out of range");
    dataset.clear();
    for (int i = 0; i < n_arrays; ++i) {
      const size_t per = inputs[i].size() / inputs[i].shape()[0];
      Storage d = B200Backend::zeros(rt::Shape{(size_t)rows, per});
      B200Backend::check(rt_memcpy_h2d(B200Backend::ctx(), d.ptr(), host_arrays[i], sizeof(float) * (size_t)rows * per));
      dataset.push_back(d);
    }
    dataset_rows = rows;
    const size_t batch = inputs[0].shape()[0];
    if (!idx_upload) B200Backend::check(rt_upload_create(B200Backend::ctx(), sizeof(int32_t) * batch, &idx_upload));
    idx_dev = B200Backend::zeros(rt::Shape{batch});
  }
  // Like step_pipelined, but the inputs are rows `indices` of the attached data set: 4 bytes per sample go to the device.
  bool step_dataset(const int64_t* indices, int64_t n, float* prev_loss) {
    if (dataset.empty()) throw Error::invalid_op("no data set attached");
    const int64_t batch = (int64_t)inputs[0].shape()[0];
    if (n != batch) throw Error(ErrorKind::DimensionMismatch, "step_dataset: one index per sample of the batch");
    pipe_setup();
    if (!graph) capture();
    rt_ctx* c = B200Backend::ctx();
    const int k = (int)(pipe_steps & 1);
    for (int64_t i = 0; i < n; ++i)
      if (indices[i] < 0 || indices[i] >= dataset_rows) throw Error(ErrorKind::InvalidIndex, "step_dataset: row outside the data set");
    // the row numbers travel like an input of step_pipelined: host -> staging on the copy stream, staging -> idx_dev by a kernel
    void* hp = nullptr;
    B200Backend::check(rt_upload_host_buffer(c, idx_upload, &hp));
    for (int64_t i = 0; i < n; ++i) static_cast<int32_t*>(hp)[i] = (int32_t)indices[i];
    void* idx_dst = idx_dev.ptr();
    B200Backend::check(rt_upload_submit_all(c, &idx_upload, &idx_dst, 1));
    for (size_t i = 0; i < inputs.size(); ++i) {
      B200Backend::make_unique(inputs[i].data_mut());
      const int64_t per = (int64_t)(inputs[i].size() / (size_t)batch);
      B200Backend::check(rt_gather_rows(c, dataset[i].ptr(), dataset_rows, per, reinterpret_cast<const int32_t*>(idx_dev.ptr()), n,
                                        inputs[i].data().ptr()));
    }
    replay();
    exchange_and_update();
    B200Backend::check(rt_publish_to_host(c, pipe_loss[k], captured_loss.data().ptr(), 1));
    B200Backend::check(rt_event_record(c, pipe_done[k]));
    const bool have_prev = pipe_steps > 0;
    if (have_prev) {
      B200Backend::check(rt_dp_wait_event(c, pipe_done[k ^ 1]));
      *prev_loss = *pipe_loss[k ^ 1];
    }
    ++pipe_steps;
    return have_prev;
  }
  float pipe_flush() {
    if (pipe_steps == 0) throw Error::invalid_op("no pipelined step has run yet");
    const int k = (int)((pipe_steps - 1) & 1);
    B200Backend::check(rt_dp_wait_event(B200Backend::ctx(), pipe_done[k]));
    return *pipe_loss[k];
  }
};

std::map<int64_t, std::shared_ptr<DpTrainer>>& dp_table() {
  static std::map<int64_t, std::shared_ptr<DpTrainer>> t;
  return t;
}
int64_t& dp_next() {
  static int64_t n = 1;
  return n;
}
DpTrainer& dp_get(int64_t h) {
  auto it = dp_table().find(h);
  if (it == dp_table().end()) throw Error::invalid_op("unknown dp trainer handle");
  return *it->second;
}

}  // namespace

extern "C" {

// Creates the device context used by every rth_* call of this process.
int rth_init(int device) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    if (B200Backend::ctx_slot()) return;
    rt_ctx* c = nullptr;
    rt_status st = rt_ctx_create(device, &c);
    if (st != RT_OK) throw Error((ErrorKind)st, "rt_ctx_create failed (no usable CUDA device?)");
    B200Backend::ctx_slot() = c;
  });
}

void* rth_ctx() { return B200Backend::ctx_slot(); }

int rth_shutdown() {
  return rt::capi::guarded<B200Backend>([&](auto& r) {
    dp_table().clear();
    r.trainers.clear();
    r.optims.clear();
    r.tensors.clear();
    if (B200Backend::ctx_slot()) {
      rt_ctx_destroy(B200Backend::ctx_slot());
      B200Backend::ctx_slot() = nullptr;
    }
  });
}

int rth_sync() {
  return rt::capi::guarded<B200Backend>([&](auto&) { B200Backend::check(rt_sync(B200Backend::ctx())); });
}

// Device pointer of a tensor's data (for calling the raw C ABI on engine tensors).
int rth_tensor_device_ptr(int64_t h, void** out) {
  return rt::capi::guarded<B200Backend>([&](auto& r) { *out = r.get(h).data().ptr(); });
}

// ---- data-parallel trainer ------------------------------------------------------------
int rth_dp_create(int config, const int64_t* dims, int nd, int rank, int world, const uint8_t* nccl_id, int64_t* out) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    auto d = std::make_shared<DpTrainer>();
    std::vector<size_t> dv(dims, dims + nd);
    d->tr = std::make_shared<rt::models::Trainer<B200Backend>>(rt::models::make_workload<B200Backend>(config, dv));
    d->rank = rank;
    d->world = world;
    if (world > 1) B200Backend::check(rt_dp_init(B200Backend::ctx(), rank, world, nccl_id));
    d->setup();
    dp_table()[dp_next()] = d;
    *out = dp_next()++;
  });
}
int rth_dp_free(int64_t h) {
  return rt::capi::guarded<B200Backend>([&](auto&) { dp_table().erase(h); });
}
int rth_dp_num_params(int64_t h, int* n) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *n = (int)dp_get(h).tr->w.params.size(); });
}
int rth_dp_param(int64_t h, int i, int64_t* out) {
  return rt::capi::guarded<B200Backend>([&](auto& r) { *out = r.put(dp_get(h).tr->w.params.at(i)); });
}
int rth_dp_input(int64_t h, int i, int64_t* out) {
  return rt::capi::guarded<B200Backend>([&](auto& r) { *out = r.put(dp_get(h).inputs.at(i)); });
}
int rth_dp_state(int64_t h, int which, int i, int64_t* out) {
  return rt::capi::guarded<B200Backend>([&](auto& r) {
    auto& d = dp_get(h);
    *out = r.put(Tensor(which == 0 ? d.state1.at(i) : d.state2.at(i), false));
  });
}
// Checkpointing: the optimizer's step counter (Adam's t) and its state tensors can be read and restored; parameters
// are restored through rth_tensor_update_from_host on the rth_dp_param handles.
int rth_dp_get_step(int64_t h, int64_t* t) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *t = dp_get(h).t; });
}
int rth_dp_set_step(int64_t h, int64_t t) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    if (t < 0 || t >= (1ll << 31)) throw Error::invalid_op("step counter out of range");
    dp_get(h).set_step(t);
  });
}
int rth_dp_set_state(int64_t h, int which, int i, const float* data, int64_t n) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    auto& d = dp_get(h);
    auto& st = which == 0 ? d.state1.at(i) : d.state2.at(i);
    B200Backend::update_from_host(st, std::vector<float>(data, data + n));
  });
}
// Diagnostic of the exchange over peer memory: the time (ns) this rank has spent waiting for its peers' gradients so far.
int rth_dp_peer_wait_ns(int64_t h, int64_t* ns) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    int words[4] = {0, 0, 0, 0};
    B200Backend::check(rt_memcpy_d2h(B200Backend::ctx(), words, dp_get(h).ctrl_ptr(), sizeof(words)));
    *ns = (int64_t)(unsigned)words[3] * 64;
  });
}
// RT_B200_DP_TRACE=1: the time stamps of the last step (ns): 0 step start, 1 forward done, 2 backward done, 3 gradients packed
// and signalled, 4 peers' gradients complete, 6 optimizer done.  Synchronises.
int rth_dp_trace(int64_t h, int64_t* out, int n) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    auto& d = dp_get(h);
    if (!d.trace.buf) throw Error::invalid_op("tracing is off (RT_B200_DP_TRACE=1 before the trainer is created)");
    std::vector<float> raw = B200Backend::copy_to_host(d.trace);
    const unsigned long long* t = reinterpret_cast<const unsigned long long*>(raw.data());
    for (int i = 0; i < n && i < 16; ++i) out[i] = (int64_t)t[i];
  });
}
// Number of floats of the flat gradient buffer: what every rank must agree on before the first exchange.
int rth_dp_flat_len(int64_t h, int64_t* n) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *n = dp_get(h).flat_len; });
}
int rth_dp_optimizer_kind(int64_t h, int* kind) {  // 0 none, 1 Adam, 2 MomentumSGD
  return rt::capi::guarded<B200Backend>([&](auto&) { *kind = dp_get(h).tr->w.optimizer; });
}
int rth_dp_set_hyper(int64_t h, const double* hp, int n) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    dp_get(h).invalidate_capture();  // a captured optimizer launch holds the old values
    auto& w = dp_get(h).tr->w;
    if (n > 0) w.lr = (float)hp[0];
    if (n > 1) w.beta1 = (float)hp[1];
    if (n > 2) w.beta2 = (float)hp[2];
    if (n > 3) w.eps = (float)hp[3];
    if (n > 4) w.momentum = (float)hp[4];
  });
}
// Pinned staging buffer of input i (fill it, then call rth_dp_step_graph with pinned = 1).
int rth_dp_pinned_input(int64_t h, int i, float** out) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *out = dp_get(h).pinned_in.at(i); });
}
int rth_dp_step_eager(int64_t h, const float* const* host_inputs, int n, float* loss) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *loss = dp_get(h).step_eager(host_inputs, n); });
}
int rth_dp_capture(int64_t h) {
  return rt::capi::guarded<B200Backend>([&](auto&) { dp_get(h).capture(); });
}
// Asynchronous: returns after enqueueing.  host_inputs may be NULL (device-resident inputs).
int rth_dp_step_graph(int64_t h, const float* const* host_inputs, int n, int pinned) {
  return rt::capi::guarded<B200Backend>([&](auto&) { dp_get(h).step_graph_async(host_inputs, n, pinned != 0); });
}
// Synchronises and returns the loss copied by the last step that uploaded inputs.
int rth_dp_last_loss(int64_t h, float* loss) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    B200Backend::check(rt_sync(B200Backend::ctx()));
    *loss = *dp_get(h).pinned_loss;
  });
}
// Pipelined steps (the host enqueues step i+1 while step i runs; the upload of step i+1 overlaps step i).
// rth_dp_pipeline_buffer: pinned buffer to fill with input i of the next step.
int rth_dp_pipeline_buffer(int64_t h, int i, float** out) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *out = dp_get(h).pipe_buffer(i); });
}
// Enqueues one step from the pipeline buffers; *has_prev tells whether *prev_loss (the previous step's loss) is valid.
int rth_dp_step_pipelined(int64_t h, float* prev_loss, int* has_prev) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *has_prev = dp_get(h).step_pipelined(prev_loss) ? 1 : 0; });
}
// Device-resident data set: rth_dp_attach_dataset uploads one [rows, sample] array per input once; rth_dp_step_dataset
// enqueues a step on the rows `indices` (gathered on the device) and returns the previous step's loss like
// rth_dp_step_pipelined.
int rth_dp_attach_dataset(int64_t h, const float* const* host_arrays, int n_arrays, int64_t rows) {
  return rt::capi::guarded<B200Backend>([&](auto&) { dp_get(h).attach_dataset(host_arrays, n_arrays, rows); });
}
int rth_dp_step_dataset(int64_t h, const int64_t* indices, int64_t n, float* prev_loss, int* has_prev) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *has_prev = dp_get(h).step_dataset(indices, n, prev_loss) ? 1 : 0; });
}
// Waits for the last pipelined step and returns its loss.
int rth_dp_pipeline_flush(int64_t h, float* loss) {
  return rt::capi::guarded<B200Backend>([&](auto&) { *loss = dp_get(h).pipe_flush(); });
}
// Peer-memory gradient exchange fused into the optimizer step (optional, world > 1, before the first step):
// every rank calls rth_dp_fused_export (192 bytes out), the handles of all ranks are gathered in rank order by the
// caller (any transport) and handed to rth_dp_fused_connect on every rank.
int rth_dp_fused_export(int64_t h, uint8_t* handles) {
  return rt::capi::guarded<B200Backend>([&](auto&) { dp_get(h).fused_export(handles); });
}
int rth_dp_fused_connect(int64_t h, const uint8_t* all_handles) {
  return rt::capi::guarded<B200Backend>([&](auto&) { dp_get(h).fused_connect(all_handles); });
}
int rth_dp_loss_tensor(int64_t h, int64_t* out) {
  return rt::capi::guarded<B200Backend>([&](auto& r) {
    auto& d = dp_get(h);
    if (!d.have_loss) throw Error::invalid_op("no step has run yet");
    *out = r.put(d.captured_loss);
  });
}
int rth_dp_graph_nodes(int64_t h, int64_t* n) {
  return rt::capi::guarded<B200Backend>([&](auto&) {
    auto& d = dp_get(h);
    *n = 0;
    if (d.graph) B200Backend::check(rt_graph_num_nodes(B200Backend::ctx(), d.graph, n));
    if (d.graph_b) {
      int64_t nb = 0;
      B200Backend::check(rt_graph_num_nodes(B200Backend::ctx(), d.graph_b, &nb));
      *n += nb;
    }
  });
}

}  // extern "C"
