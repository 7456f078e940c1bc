// Node-API addon: forwards the calls of jax_js_b200/ts/cuda.ts to libjaxcuda.so (include/jaxcuda.h).
// Build where Node headers exist:
//   g++ -std=c++17 -shared -fPIC -I$(node -p "require('node-addon-api').include_dir") -I<node>/include/node \
//       -Iinclude addon.cc -Ljax_js_b200 -ljaxcuda -Wl,-rpath,'$ORIGIN' -o jaxcuda_addon.node
// Not compiled in this repository: the build image has neither Node nor node_api.h.
#include <napi.h>

#include <cstring>
#include <map>
#include <vector>

#include "jaxcuda.h"

namespace {

jaxcuda_ctx* Ctx(const Napi::Value& v) {
  bool lossless;
  return reinterpret_cast<jaxcuda_ctx*>(v.As<Napi::BigInt>().Uint64Value(&lossless));
}
jaxcuda_exe* Exe(const Napi::Value& v) {
  bool lossless;
  return reinterpret_cast<jaxcuda_exe*>(v.As<Napi::BigInt>().Uint64Value(&lossless));
}
Napi::Value Handle(Napi::Env env, void* p) { return Napi::BigInt::New(env, (uint64_t)(uintptr_t)p); }

void Throw(Napi::Env env, jaxcuda_ctx* ctx) { throw Napi::Error::New(env, jaxcuda_last_error(ctx)); }

Napi::Value Create(const Napi::CallbackInfo& info) {
  jaxcuda_ctx* ctx = nullptr;
  if (jaxcuda_create(info[0].As<Napi::Number>().Int32Value(), &ctx) != JAXCUDA_OK) Throw(info.Env(), nullptr);
  return Handle(info.Env(), ctx);
}
void Destroy(const Napi::CallbackInfo& info) { jaxcuda_destroy(Ctx(info[0])); }
Napi::Value LastError(const Napi::CallbackInfo& info) { return Napi::String::New(info.Env(), jaxcuda_last_error(Ctx(info[0]))); }

Napi::Value Malloc(const Napi::CallbackInfo& info) {
  jaxcuda_ctx* ctx = Ctx(info[0]);
  const size_t bytes = (size_t)info[1].As<Napi::Number>().Int64Value();
  const void* init = nullptr;
  size_t init_bytes = 0;
  if (info.Length() > 2 && info[2].IsTypedArray()) {
    auto a = info[2].As<Napi::Uint8Array>();
    init = a.Data();
    init_bytes = a.ByteLength();
  }
  jaxcuda_slot slot = 0;
  if (jaxcuda_malloc(ctx, bytes, init, init_bytes, &slot) != JAXCUDA_OK) Throw(info.Env(), ctx);
  return Napi::Number::New(info.Env(), slot);
}
Napi::Value IncRef(const Napi::CallbackInfo& info) {
  return Napi::Number::New(info.Env(), jaxcuda_incref(Ctx(info[0]), info[1].As<Napi::Number>().Uint32Value()));
}
Napi::Value DecRef(const Napi::CallbackInfo& info) {
  return Napi::Number::New(info.Env(), jaxcuda_decref(Ctx(info[0]), info[1].As<Napi::Number>().Uint32Value()));
}
Napi::Value Read(const Napi::CallbackInfo& info) {
  jaxcuda_ctx* ctx = Ctx(info[0]);
  const jaxcuda_slot slot = info[1].As<Napi::Number>().Uint32Value();
  const size_t start = (size_t)info[2].As<Napi::Number>().Int64Value();
  int64_t count = info[3].As<Napi::Number>().Int64Value();
  size_t size = 0;
  if (jaxcuda_slot_size(ctx, slot, &size) != JAXCUDA_OK) Throw(info.Env(), ctx);
  if (count < 0) count = (int64_t)(size - start);
  auto out = Napi::Uint8Array::New(info.Env(), (size_t)count);
  if (jaxcuda_read(ctx, slot, start, (size_t)count, out.Data()) != JAXCUDA_OK) Throw(info.Env(), ctx);
  return out;
}
// Backend.read as a Promise.  The copy is enqueued on the library's download stream into pinned
// memory right away (ordered after the dispatches so far).  One host thread drives a context at a
// time, so the worker thread never enters the context: it blocks on the ticket's event alone
// (jaxcuda_event_block), and the ticket is retired, the result copied and the staging buffer
// recycled back on the JS thread.
class PinnedPool {  // staging buffers by capacity: allocating pinned memory synchronises the device, so they are kept
 public:
  void* Get(jaxcuda_ctx* ctx, size_t bytes, size_t* capacity) {
    size_t cap = 4096;
    while (cap < bytes) cap <<= 1;
    *capacity = cap;
    auto& list = free_[cap];
    if (!list.empty()) { void* p = list.back(); list.pop_back(); return p; }
    void* p = nullptr;
    return jaxcuda_host_alloc(ctx, cap, &p) == JAXCUDA_OK ? p : nullptr;
  }
  void Put(size_t capacity, void* p) { free_[capacity].push_back(p); }

 private:
  std::map<size_t, std::vector<void*>> free_;
};
static PinnedPool g_pinned;   // used on the JS thread only

class ReadWorker : public Napi::AsyncWorker {
 public:
  ReadWorker(Napi::Env env, jaxcuda_ctx* ctx, jaxcuda_slot slot, void* pinned, size_t capacity, size_t count, uint64_t ticket,
             void* event)
      : Napi::AsyncWorker(env), deferred_(Napi::Promise::Deferred::New(env)), ctx_(ctx), slot_(slot), pinned_(pinned),
        capacity_(capacity), count_(count), ticket_(ticket), event_(event) {}
  Napi::Promise Promise() const { return deferred_.Promise(); }
  void Execute() override {   // worker thread: no context state is touched here
    if (jaxcuda_event_block(event_) != JAXCUDA_OK) SetError("waiting for the device-to-host copy failed");
  }
  void OnOK() override {      // JS thread
    const int rc = jaxcuda_read_wait(ctx_, ticket_);   // returns at once; reports a kernel that gave up a bounded wait
    auto out = Napi::Uint8Array::New(Env(), count_);
    if (count_) memcpy(out.Data(), pinned_, count_);
    Release();
    if (rc == JAXCUDA_OK) deferred_.Resolve(out);
    else deferred_.Reject(Napi::Error::New(Env(), jaxcuda_last_error(ctx_)).Value());
  }
  void OnError(const Napi::Error& e) override {
    jaxcuda_read_wait(ctx_, ticket_);
    Release();
    deferred_.Reject(e.Value());
  }

 private:
  void Release() {
    g_pinned.Put(capacity_, pinned_);
    jaxcuda_decref(ctx_, slot_);           // the reference taken in ReadAsync kept the buffer alive
  }
  Napi::Promise::Deferred deferred_;
  jaxcuda_ctx* ctx_;
  jaxcuda_slot slot_;
  void* pinned_;
  size_t capacity_, count_;
  uint64_t ticket_;
  void* event_;
};
Napi::Value ReadAsync(const Napi::CallbackInfo& info) {
  jaxcuda_ctx* ctx = Ctx(info[0]);
  const jaxcuda_slot slot = info[1].As<Napi::Number>().Uint32Value();
  const size_t start = (size_t)info[2].As<Napi::Number>().Int64Value();
  int64_t count = info[3].As<Napi::Number>().Int64Value();
  size_t size = 0;
  if (jaxcuda_slot_size(ctx, slot, &size) != JAXCUDA_OK) Throw(info.Env(), ctx);
  if (count < 0) count = (int64_t)(size - start);
  size_t capacity = 0;
  void* pinned = g_pinned.Get(ctx, (size_t)count, &capacity);
  if (!pinned) Throw(info.Env(), ctx);
  uint64_t ticket = 0;
  void* event = nullptr;
  jaxcuda_incref(ctx, slot);               // a caller may drop its reference before the Promise resolves
  if (jaxcuda_read_async(ctx, slot, start, (size_t)count, pinned, &ticket) != JAXCUDA_OK ||
      jaxcuda_read_event(ctx, ticket, &event) != JAXCUDA_OK) {
    jaxcuda_decref(ctx, slot);
    g_pinned.Put(capacity, pinned);
    Throw(info.Env(), ctx);
  }
  auto* worker = new ReadWorker(info.Env(), ctx, slot, pinned, capacity, (size_t)count, ticket, event);
  worker->Queue();
  return worker->Promise();
}
Napi::Value PrepareKernel(const Napi::CallbackInfo& info) {
  jaxcuda_ctx* ctx = Ctx(info[0]);
  auto image = info[1].As<Napi::Uint8Array>();
  bool lossless;
  const uint64_t hash = info[2].As<Napi::BigInt>().Uint64Value(&lossless);
  jaxcuda_exe* exe = nullptr;
  if (jaxcuda_prepare_kernel(ctx, image.Data(), image.ByteLength(), hash, &exe) != JAXCUDA_OK) Throw(info.Env(), ctx);
  return Handle(info.Env(), exe);
}
Napi::Value PrepareRoutine(const Napi::CallbackInfo& info) {
  jaxcuda_ctx* ctx = Ctx(info[0]);
  const std::string name = info[1].As<Napi::String>();
  auto type = info[2].As<Napi::Object>();
  static const char* kDtypes[] = {"float32", "int32", "uint32", "bool", "float16", "float64"};
  auto dtypes = [&](const char* key, std::vector<int32_t>& out) {
    auto arr = type.Get(key).As<Napi::Array>();
    for (uint32_t i = 0; i < arr.Length(); i++) {
      const std::string s = arr.Get(i).As<Napi::String>();
      for (int d = 0; d < 6; d++) if (s == kDtypes[d]) out.push_back(d);
    }
  };
  auto shapes = [&](const char* key, std::vector<int32_t>& ranks, std::vector<int64_t>& flat) {
    auto arr = type.Get(key).As<Napi::Array>();
    for (uint32_t i = 0; i < arr.Length(); i++) {
      auto shape = arr.Get(i).As<Napi::Array>();
      ranks.push_back((int32_t)shape.Length());
      for (uint32_t j = 0; j < shape.Length(); j++) flat.push_back(shape.Get(j).As<Napi::Number>().Int64Value());
    }
  };
  std::vector<int32_t> idt, odt, irk, ork;
  std::vector<int64_t> ish, osh;
  dtypes("inputDtypes", idt); dtypes("outputDtypes", odt);
  shapes("inputShapes", irk, ish); shapes("outputShapes", ork, osh);
  jaxcuda_routine_type rt{(int)irk.size(), (int)ork.size(), idt.data(), irk.data(), ish.data(), odt.data(), ork.data(), osh.data()};
  const std::string params = info[3].As<Napi::String>();
  jaxcuda_exe* exe = nullptr;
  if (jaxcuda_prepare_routine(ctx, name.c_str(), &rt, params.c_str(), &exe) != JAXCUDA_OK) Throw(info.Env(), ctx);
  return Handle(info.Env(), exe);
}
Napi::Value Dispatch(const Napi::CallbackInfo& info) {
  auto in = info[2].As<Napi::Uint32Array>(), out = info[3].As<Napi::Uint32Array>();
  return Napi::Number::New(info.Env(), jaxcuda_dispatch(Ctx(info[0]), Exe(info[1]), in.Data(), (int)in.ElementLength(),
                                                        out.Data(), (int)out.ElementLength()));
}

jaxcuda_graph* Graph(const Napi::Value& v) {
  bool lossless;
  return reinterpret_cast<jaxcuda_graph*>((uintptr_t)v.As<Napi::BigInt>().Uint64Value(&lossless));
}

// Replay of a static step list as one CUDA graph (the counterpart of JitProgram.execute,
// src/frontend/jit.ts:111-162): between captureBegin and captureEnd the calls above are recorded.
Napi::Value CaptureBegin(const Napi::CallbackInfo& info) {
  if (jaxcuda_capture_begin(Ctx(info[0])) != JAXCUDA_OK) Throw(info.Env(), Ctx(info[0]));
  return info.Env().Undefined();
}
Napi::Value CaptureEnd(const Napi::CallbackInfo& info) {
  jaxcuda_graph* graph = nullptr;
  if (jaxcuda_capture_end(Ctx(info[0]), &graph) != JAXCUDA_OK) Throw(info.Env(), Ctx(info[0]));
  return Handle(info.Env(), graph);
}
Napi::Value GraphLaunch(const Napi::CallbackInfo& info) {
  jaxcuda_graph* graph = Graph(info[1]);
  if (jaxcuda_graph_launch(Ctx(info[0]), graph) != JAXCUDA_OK) Throw(info.Env(), Ctx(info[0]));
  return info.Env().Undefined();
}
Napi::Value GraphDestroy(const Napi::CallbackInfo& info) {
  jaxcuda_graph* graph = Graph(info[1]);
  if (jaxcuda_graph_destroy(Ctx(info[0]), graph) != JAXCUDA_OK) Throw(info.Env(), Ctx(info[0]));
  return info.Env().Undefined();
}
Napi::Value GraphCost(const Napi::CallbackInfo& info) {   // what JitProgram.toString() would print about the replay
  jaxcuda_graph* graph = Graph(info[0]);
  uint64_t launches = 0;
  double bytes = 0;
  int fused = 0;
  jaxcuda_graph_cost(graph, &launches, &bytes, &fused);
  auto out = Napi::Object::New(info.Env());
  out.Set("launches", Napi::Number::New(info.Env(), (double)launches));
  out.Set("bytes", Napi::Number::New(info.Env(), bytes));
  out.Set("fusedRuns", Napi::Number::New(info.Env(), fused));
  return out;
}

// Per-dispatch timing while the reference's profiler is on (src/tracing.ts:15-33).
Napi::Value TraceStart(const Napi::CallbackInfo& info) {
  if (jaxcuda_trace_start(Ctx(info[0])) != JAXCUDA_OK) Throw(info.Env(), Ctx(info[0]));
  return info.Env().Undefined();
}
Napi::Value TraceStop(const Napi::CallbackInfo& info) {
  int n = 0;
  if (jaxcuda_trace_stop(Ctx(info[0]), &n) != JAXCUDA_OK) Throw(info.Env(), Ctx(info[0]));
  auto out = Napi::Array::New(info.Env(), n);
  for (int i = 0; i < n; i++) {
    double start = 0, duration = 0;
    if (jaxcuda_trace_record(Ctx(info[0]), i, nullptr, &start, &duration, nullptr, 0) != JAXCUDA_OK) Throw(info.Env(), Ctx(info[0]));
    auto rec = Napi::Object::New(info.Env());
    rec.Set("startMs", Napi::Number::New(info.Env(), start));
    rec.Set("durationMs", Napi::Number::New(info.Env(), duration));
    out.Set((uint32_t)i, rec);
  }
  return out;
}

Napi::Object Init(Napi::Env env, Napi::Object exports) {
  exports.Set("create", Napi::Function::New(env, Create));
  exports.Set("destroy", Napi::Function::New(env, Destroy));
  exports.Set("lastError", Napi::Function::New(env, LastError));
  exports.Set("malloc", Napi::Function::New(env, Malloc));
  exports.Set("incref", Napi::Function::New(env, IncRef));
  exports.Set("decref", Napi::Function::New(env, DecRef));
  exports.Set("read", Napi::Function::New(env, Read));
  exports.Set("readAsync", Napi::Function::New(env, ReadAsync));
  exports.Set("prepareKernel", Napi::Function::New(env, PrepareKernel));
  exports.Set("prepareRoutine", Napi::Function::New(env, PrepareRoutine));
  exports.Set("dispatch", Napi::Function::New(env, Dispatch));
  exports.Set("captureBegin", Napi::Function::New(env, CaptureBegin));
  exports.Set("captureEnd", Napi::Function::New(env, CaptureEnd));
  exports.Set("graphLaunch", Napi::Function::New(env, GraphLaunch));
  exports.Set("graphDestroy", Napi::Function::New(env, GraphDestroy));
  exports.Set("graphCost", Napi::Function::New(env, GraphCost));
  exports.Set("traceStart", Napi::Function::New(env, TraceStart));
  exports.Set("traceStop", Napi::Function::New(env, TraceStop));
  return exports;
}

}  // namespace

NODE_API_MODULE(jaxcuda_addon, Init)
