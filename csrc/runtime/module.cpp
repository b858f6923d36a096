#include "module.h"

#include <cstring>
#include <fstream>
#include <sstream>

#include "../kernels/gemm_args.h"

namespace spike {

static std::string read_file(const std::string& path, bool binary) {
  std::ifstream f(path, binary ? std::ios::binary : std::ios::in);
  if (!f) throw SpikeError("cannot open '" + path + "'");
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

static std::string sidecar_path(const std::string& cubin_path) {
  size_t dot = cubin_path.rfind('.');
  std::string stem = dot == std::string::npos ? cubin_path : cubin_path.substr(0, dot);
  return stem + ".json";
}

LoadedModule::LoadedModule(const CudaRuntime& rt, const std::string& path, int core_id, bool cc_enabled, int rank_id,
                           int world_size)
    : rt_(rt), path_(path), core_id_(core_id), rank_id_(rank_id), world_size_(world_size), cc_enabled_(cc_enabled),
      runtime_closed_(rt.closed_token()) {
  if (core_id != 0 && core_id != rt.device_ordinal())
    throw SpikeError("core_id " + std::to_string(core_id) + " is not the device this process drives");
  if (cc_enabled && (rank_id < 0 || world_size < 1 || rank_id >= world_size))
    throw SpikeError("collective load needs 0 <= rank_id < world_size");
  rt.make_current();
  const Driver& d = driver();
  const std::string image = read_file(path, true);
  const Json plan = Json::parse(read_file(sidecar_path(path), false));
  name_ = plan.has("name") ? plan.at("name").as_string() : "kernel";
  check(d.cuModuleLoadData(&module_, image.data()), "cuModuleLoadData");

  const Json& bufs = plan.at("buffers");
  bufs_.resize(bufs.size());
  for (size_t i = 0; i < bufs.size(); ++i) {
    const Json& b = bufs.at(i);
    Buf& dst = bufs_[b.at("index").as_int()];
    dst.nbytes = static_cast<size_t>(b.at("nbytes").as_int());
    dst.kind = b.at("kind").as_string();
    dst.name = b.at("name").as_string();
    if (b.has("alias_of")) dst.alias_of = static_cast<int>(b.at("alias_of").as_int());
    if (dst.kind == "temp" || dst.kind == "const") {
      check(d.cuMemAlloc_v2(&dst.owned, dst.nbytes ? dst.nbytes : 1), "cuMemAlloc(plan buffer)");
      if (dst.kind == "const") {
        std::vector<uint8_t> data = base64_decode(b.at("data").as_string());
        if (data.size() > dst.nbytes) throw SpikeError("constant larger than its buffer in plan of " + path);
        if (!data.empty()) check(d.cuMemcpyHtoD_v2(dst.owned, data.data(), data.size()), "cuMemcpyHtoD(const)");
      }
    }
  }
  auto meta = [](const Json& t) {
    TensorMetadata m;
    m.dtype = t.at("dtype").as_string();
    size_t n = 1;
    for (size_t i = 0; i < t.at("shape").size(); ++i) {
      m.shape.push_back(t.at("shape").at(i).as_int());
      n *= static_cast<size_t>(t.at("shape").at(i).as_int());
    }
    static const std::map<std::string, size_t> width = {
        {"pred", 1}, {"i8", 1}, {"u8", 1}, {"f8e5m2", 1}, {"f8e4m3", 1}, {"i16", 2}, {"u16", 2}, {"f16", 2},
        {"bf16", 2}, {"i32", 4}, {"u32", 4}, {"f32", 4}, {"i64", 8}, {"u64", 8}, {"f64", 8}};
    auto it = width.find(m.dtype);
    if (it == width.end()) throw SpikeError("unknown dtype '" + m.dtype + "' in plan");
    m.size = n * it->second;
    return m;
  };
  for (size_t i = 0; i < plan.at("inputs").size(); ++i) {
    const Json& t = plan.at("inputs").at(i);
    const std::string nm = t.at("name").as_string();
    info_.inputs[nm] = meta(t);
    info_.input_order.push_back(nm);
    input_buf_[nm] = static_cast<int>(t.at("buffer").as_int());
  }
  for (size_t i = 0; i < plan.at("outputs").size(); ++i) {
    const Json& t = plan.at("outputs").at(i);
    const std::string nm = t.at("name").as_string();
    info_.outputs[nm] = meta(t);
    info_.output_order.push_back(nm);
    const int bi = static_cast<int>(t.at("buffer").as_int());
    output_buf_[nm] = bi;
    if (bufs_[bi].alias_of >= 0) {
      for (auto& kv : input_buf_)
        if (kv.second == bufs_[bi].alias_of) info_.aliases[nm] = kv.first;
    }
  }
  const Json& ls = plan.at("launches");
  for (size_t i = 0; i < ls.size(); ++i) {
    const Json& l = ls.at(i);
    LaunchRec rec;
    rec.kernel = l.at("kernel").as_string();
    if (l.has("loc") && !l.at("loc").is_null()) rec.loc = l.at("loc").as_string();
    for (int k = 0; k < 3; ++k) {
      rec.grid[k] = static_cast<unsigned>(l.at("grid").at(k).as_int());
      rec.block[k] = static_cast<unsigned>(l.at("block").at(k).as_int());
    }
    rec.smem = static_cast<unsigned>(l.at("smem").as_int());
    check(d.cuModuleGetFunction(&rec.fn, module_, rec.kernel.c_str()), ("cuModuleGetFunction(" + rec.kernel + ")").c_str());
    if (rec.smem > 48 * 1024)
      check(d.cuFuncSetAttribute(rec.fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, static_cast<int>(rec.smem)),
            "cuFuncSetAttribute(smem)");
    for (size_t a = 0; a < l.at("args").size(); ++a) {
      const Json& ja = l.at("args").at(a);
      Arg arg;
      if (ja.has("buffer")) {
        arg.kind = Arg::Buffer;
        arg.buffer = static_cast<int>(ja.at("buffer").as_int());
        arg.offset = ja.has("offset") ? ja.at("offset").as_int() : 0;
      } else if (ja.has("i32")) {
        arg.kind = Arg::I32;
        arg.ival = ja.at("i32").as_int();
      } else if (ja.has("i64")) {
        arg.kind = Arg::I64;
        arg.ival = ja.at("i64").as_int();
      } else if (ja.has("f32")) {
        arg.kind = Arg::F32;
        arg.fval = ja.at("f32").as_double();
      } else if (ja.has("tensormap")) {
        const Json& tm = ja.at("tensormap");
        arg.kind = Arg::TensorMap;
        arg.buffer = static_cast<int>(tm.at("buffer").as_int());
        arg.offset = tm.at("offset").as_int();
        for (size_t k = 0; k < tm.at("dims").size(); ++k) arg.dims.push_back(tm.at("dims").at(k).as_int());
        for (size_t k = 0; k < tm.at("strides").size(); ++k) arg.strides.push_back(tm.at("strides").at(k).as_int());
        for (size_t k = 0; k < tm.at("box").size(); ++k) arg.box.push_back(static_cast<unsigned>(tm.at("box").at(k).as_int()));
      } else if (ja.has("gemm_args")) {
        arg.kind = Arg::GemmArgs;
        arg.gemm = ja.at("gemm_args");
      } else if (ja.has("cc")) {
        arg.kind = Arg::CcTable;
      } else {
        throw SpikeError("unknown launch argument kind in plan of " + path);
      }
      rec.args.push_back(std::move(arg));
    }
    launches_.push_back(std::move(rec));
  }
  if (plan.has("collective")) {
    const Json& c = plan.at("collective");
    cc_world_ = static_cast<int>(c.at("world").as_int());
    cc_half_bytes_ = static_cast<size_t>(c.at("half_bytes").as_int());
    cc_workspace_bytes_ = static_cast<size_t>(c.at("workspace_bytes").as_int());
    if (cc_world_ > 1 && (!cc_enabled || world_size != cc_world_))
      throw SpikeError("'" + path + "' contains collectives over " + std::to_string(cc_world_) +
                       " ranks: load it with cc_enabled and world_size " + std::to_string(cc_world_));
    if (cc_world_ == 1) {
      // traced for a single rank: the only peer is this process
      check(d.cuMemAlloc_v2(&cc_private_ws_, cc_workspace_bytes_), "cuMemAlloc(collective workspace)");
      check(d.cuMemsetD8_v2(cc_private_ws_, 0, cc_workspace_bytes_), "cuMemsetD8(collective workspace)");
      set_collective_workspace({static_cast<unsigned long long>(cc_private_ws_)});
    }
  }
}

namespace {
// Must match `CcTable` in the prelude of the generated source (nkipy_b200/compiler/codegen.py).
struct CcTableHost {
  unsigned long long peer_ws[8];
  unsigned long long local_ws;
  unsigned long long seen;
  unsigned long long done;
  unsigned long long status;
  long long half_bytes;
  int rank, world;
};
}  // namespace

void LoadedModule::set_collective_workspace(const std::vector<unsigned long long>& peer_ws) {
  if (!module_) throw SpikeError("model '" + name_ + "' was unloaded");
  if (cc_world_ <= 0) throw SpikeError("'" + name_ + "' has no collectives");
  if (static_cast<int>(peer_ws.size()) != cc_world_)
    throw SpikeError("collective workspace table needs " + std::to_string(cc_world_) + " entries");
  if (cc_table_) throw SpikeError("collective workspace of '" + name_ + "' is already set");
  const int rank = cc_world_ == 1 ? 0 : rank_id_;
  rt_.make_current();
  const Driver& d = driver();
  check(d.cuMemAlloc_v2(&cc_counters_, 64), "cuMemAlloc(collective counters)");
  check(d.cuMemsetD8_v2(cc_counters_, 0, 64), "cuMemsetD8(collective counters)");
  CcTableHost t{};
  for (int i = 0; i < cc_world_; ++i) t.peer_ws[i] = peer_ws[i];
  t.local_ws = peer_ws[rank];
  t.seen = static_cast<unsigned long long>(cc_counters_);
  t.done = static_cast<unsigned long long>(cc_counters_) + 16;
  t.status = reinterpret_cast<unsigned long long>(rt_.status_word());
  t.half_bytes = static_cast<long long>(cc_half_bytes_);
  t.rank = rank;
  t.world = cc_world_;
  check(d.cuMemAlloc_v2(&cc_table_, sizeof(t)), "cuMemAlloc(collective table)");
  check(d.cuMemcpyHtoD_v2(cc_table_, &t, sizeof(t)), "cuMemcpyHtoD(collective table)");
}

void LoadedModule::unload() {
  if (!module_) return;
  if (!runtime_closed_->load()) {
    const Driver& d = driver();
    rt_.make_current();
    for (auto& b : bufs_)
      if (b.owned) d.cuMemFree_v2(b.owned);
    if (cc_table_) d.cuMemFree_v2(cc_table_);
    if (cc_counters_) d.cuMemFree_v2(cc_counters_);
    if (cc_private_ws_) d.cuMemFree_v2(cc_private_ws_);
    d.cuModuleUnload(module_);
  }
  for (auto& b : bufs_) b.owned = 0;
  cc_table_ = cc_counters_ = cc_private_ws_ = 0;
  module_ = nullptr;
}

LoadedModule::~LoadedModule() {
  try {
    unload();
  } catch (...) {
  }
}

void LoadedModule::execute(const TensorSet& inputs, const TensorSet& outputs, const std::string& trace_path,
                           bool save_trace) {
  if (!module_) throw SpikeError("model '" + name_ + "' was unloaded");
  if (runtime_closed_->load()) throw SpikeError("runtime is closed");
  if (cc_world_ > 0 && !cc_table_)
    throw SpikeError("'" + name_ + "' contains collectives: call set_collective_workspace with the ranks' symmetric "
                     "workspaces before the first execute");
  rt_.make_current();
  const Driver& d = driver();
  CUstream stream = rt_.stream();
  // ---- bind buffers
  std::vector<CUdeviceptr> ptr(bufs_.size(), 0);
  for (size_t i = 0; i < bufs_.size(); ++i) ptr[i] = bufs_[i].owned;
  for (auto& kv : input_buf_) {
    auto t = inputs.get(kv.first);
    if (t->is_freed()) throw SpikeError("input tensor '" + kv.first + "' was freed");
    if (t->size() < bufs_[kv.second].nbytes)
      throw SpikeError("input tensor '" + kv.first + "' has " + std::to_string(t->size()) + " bytes, kernel needs " +
                       std::to_string(bufs_[kv.second].nbytes));
    ptr[kv.second] = t->ptr();
  }
  std::vector<std::pair<int, int>> write_back;   // (output buffer, aliased input buffer) when they differ
  for (auto& kv : output_buf_) {
    auto t = outputs.get(kv.first);
    if (t->is_freed()) throw SpikeError("output tensor '" + kv.first + "' was freed");
    if (t->size() < bufs_[kv.second].nbytes)
      throw SpikeError("output tensor '" + kv.first + "' has " + std::to_string(t->size()) + " bytes, kernel needs " +
                       std::to_string(bufs_[kv.second].nbytes));
    ptr[kv.second] = t->ptr();
  }
  // An aliased output that was given the same memory as its input is computed into a scratch
  // allocation and copied back after the launches (generated kernels read the old contents
  // while writing the new ones).
  std::vector<CUdeviceptr> scratch;
  for (size_t i = 0; i < bufs_.size(); ++i) {
    const int a = bufs_[i].alias_of;
    if (a >= 0 && ptr[i] == ptr[a]) {
      CUdeviceptr tmp = 0;
      check(d.cuMemAlloc_v2(&tmp, bufs_[i].nbytes ? bufs_[i].nbytes : 1), "cuMemAlloc(alias scratch)");
      scratch.push_back(tmp);
      ptr[i] = tmp;
      write_back.emplace_back(static_cast<int>(i), a);
    }
  }
  TraceSession* session = TraceSession::current();
  const bool timed = save_trace || session != nullptr;
  std::vector<CUevent> ev;
  if (timed) {
    ev.resize(launches_.size() + 1);
    for (auto& e : ev) check(d.cuEventCreate(&e, CU_EVENT_DEFAULT), "cuEventCreate");
    check(d.cuEventRecord(ev[0], stream), "cuEventRecord");
  }
  // ---- launches
  for (size_t li = 0; li < launches_.size(); ++li) {
    LaunchRec& l = launches_[li];
    std::vector<std::vector<uint8_t>> storage;
    storage.reserve(l.args.size());
    for (const Arg& a : l.args) {
      switch (a.kind) {
        case Arg::Buffer: {
          CUdeviceptr p = ptr[a.buffer] + static_cast<CUdeviceptr>(a.offset);
          storage.emplace_back(sizeof(p));
          std::memcpy(storage.back().data(), &p, sizeof(p));
          break;
        }
        case Arg::I32: {
          int v = static_cast<int>(a.ival);
          storage.emplace_back(sizeof(v));
          std::memcpy(storage.back().data(), &v, sizeof(v));
          break;
        }
        case Arg::I64: {
          long long v = a.ival;
          storage.emplace_back(sizeof(v));
          std::memcpy(storage.back().data(), &v, sizeof(v));
          break;
        }
        case Arg::F32: {
          float v = static_cast<float>(a.fval);
          storage.emplace_back(sizeof(v));
          std::memcpy(storage.back().data(), &v, sizeof(v));
          break;
        }
        case Arg::TensorMap: {
          // CUtensorMap must be 64-byte aligned: over-allocate and align inside the vector
          storage.emplace_back(sizeof(CUtensorMap) + 64);
          uint8_t* base = storage.back().data();
          CUtensorMap* tm = reinterpret_cast<CUtensorMap*>((reinterpret_cast<uintptr_t>(base) + 63) & ~uintptr_t(63));
          cuuint64_t dims[5], strides[5];
          cuuint32_t box[5], estr[5];
          const cuuint32_t rank = static_cast<cuuint32_t>(a.dims.size());
          for (cuuint32_t k = 0; k < rank; ++k) {
            dims[k] = a.dims[k];
            box[k] = a.box[k];
            estr[k] = 1;
            if (k + 1 < rank) strides[k] = a.strides[k];
          }
          check(d.cuTensorMapEncodeTiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank,
                                         reinterpret_cast<void*>(ptr[a.buffer] + static_cast<CUdeviceptr>(a.offset)),
                                         dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                "cuTensorMapEncodeTiled");
          break;
        }
        case Arg::CcTable: {
          CUdeviceptr p = cc_table_;
          storage.emplace_back(sizeof(p));
          std::memcpy(storage.back().data(), &p, sizeof(p));
          break;
        }
        case Arg::GemmArgs: {
          nkb::GemmArgs g{};
          const Json& j = a.gemm;
          g.rows = static_cast<int>(j.at("rows").as_int());
          g.cols = static_cast<int>(j.at("cols").as_int());
          g.k = static_cast<int>(j.at("k").as_int());
          g.kb_total = (g.k + nkb::kBlockK - 1) / nkb::kBlockK;
          g.splits = 1;
          g.kb_per_split = g.kb_total;
          const int bn = static_cast<int>(j.at("block_n").as_int());
          g.num_row_tiles = (g.rows + nkb::kTileRows - 1) / nkb::kTileRows;
          g.num_col_tiles = (g.cols + bn - 1) / bn;
          g.stages = static_cast<int>(j.at("stages").as_int());
          g.weights_operand = -1;
          g.ldo = j.at("ldo").as_int();
          g.out = reinterpret_cast<void*>(ptr[j.at("out_buffer").as_int()] + static_cast<CUdeviceptr>(j.at("out_offset").as_int()));
          g.status = rt_.status_word();
          storage.emplace_back(sizeof(g));
          std::memcpy(storage.back().data(), &g, sizeof(g));
          // the kernel also takes the (empty) peer-push block
          storage.emplace_back(sizeof(nkb::PushArgs));
          std::memset(storage.back().data(), 0, sizeof(nkb::PushArgs));
          break;
        }
      }
    }
    // kernel parameter pointers, in declaration order (a GEMM block is followed by its push block)
    std::vector<void*> ordered;
    {
      size_t si = 0;
      ordered.reserve(l.args.size() + 1);
      for (const Arg& a : l.args) {
        if (a.kind == Arg::TensorMap) {
          uint8_t* base = storage[si].data();
          ordered.push_back(reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(base) + 63) & ~uintptr_t(63)));
          ++si;
        } else if (a.kind == Arg::GemmArgs) {
          ordered.push_back(storage[si].data());
          ordered.push_back(storage[si + 1].data());
          si += 2;
        } else {
          ordered.push_back(storage[si].data());
          ++si;
        }
      }
    }
    check(d.cuLaunchKernel(l.fn, l.grid[0], l.grid[1], l.grid[2], l.block[0], l.block[1], l.block[2], l.smem, stream,
                           ordered.data(), nullptr),
          ("cuLaunchKernel(" + l.kernel + ")").c_str());
    if (timed) check(d.cuEventRecord(ev[li + 1], stream), "cuEventRecord");
  }
  for (auto& wb : write_back)
    check(d.cuMemcpyDtoDAsync_v2(ptr[wb.second], ptr[wb.first], bufs_[wb.first].nbytes, stream), "cuMemcpyDtoD(alias)");
  CUresult sync = d.cuStreamSynchronize(stream);
  for (CUdeviceptr s : scratch) d.cuMemFree_v2(s);
  check(sync, ("execute of '" + name_ + "'").c_str());
  const int status = rt_.read_status(true);
  if (status)
    throw SpikeRuntimeError("kernel '" + name_ + "' reported device status " + std::to_string(status & 0xFF) +
                            " (a bounded wait inside a kernel gave up)");
  if (timed) {
    std::vector<double> ms(launches_.size(), 0.0);
    double total = 0;
    for (size_t li = 0; li < launches_.size(); ++li) {
      float t = 0;
      d.cuEventElapsedTime(&t, ev[li], ev[li + 1]);
      ms[li] = t;
      total += t;
    }
    if (session) {
      static double clock_ns = 0;   // monotonically increasing device-time axis for the session
      const long long id = session->next_tracking_id();
      session->record({"kernel_exec", "start", id, clock_ns, core_id_, name_});
      clock_ns += total * 1e6;
      session->record({"kernel_exec", "stop", id, clock_ns, core_id_, name_});
    }
    if (save_trace && !trace_path.empty()) {
      std::ofstream out(trace_path);
      out.precision(9);
      out << "{\"model\": " << Json::quote(name_) << ", \"total_ms\": " << total << ", \"launches\": [";
      for (size_t li = 0; li < launches_.size(); ++li) {
        if (li) out << ", ";
        out << "{\"kernel\": " << Json::quote(launches_[li].kernel) << ", \"ms\": " << ms[li]
            << ", \"loc\": " << Json::quote(launches_[li].loc) << "}";
      }
      out << "]}\n";
    }
    for (auto& e : ev) d.cuEventDestroy_v2(e);
  }
}

}  // namespace spike
