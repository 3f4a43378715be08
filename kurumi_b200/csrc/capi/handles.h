// Opaque C-ABI handle layouts and the error/exception guard shared by every extern "C" entry.
// Mirrors kurumi/src/capi.rs:26-112: heap-allocated newtypes, a thread-local last-error string,
// and a guard that turns any failure inside a builder into the sentinel return value.
#pragma once
#include <memory>
#include <string>

#include "../core/graph.h"
#include "../core/serialize.h"

struct KuGraph { ku::Graph g; };
struct KuTensor { ku::TensorPtr t; };
struct KuFeeds { ku::Feeds f; };
struct KuBackend { std::unique_ptr<ku::Backend> b; };
struct KuRunnable { ku::Runnable r; };
struct KuPlan { std::shared_ptr<ku::Backend> backend; uint64_t graph_id; ku::NodeId node; };

namespace ku {
void set_err(const std::string& msg);

// Run f at the boundary; any exception becomes `on_err` with the message stored for
// ku_last_error(). The process is never aborted by a bad argument.
template <typename T, typename F>
T guard(T on_err, F&& f) {
  try {
    return f();
  } catch (const std::exception& e) {
    set_err(e.what());
  } catch (...) {
    set_err("panic at FFI boundary");
  }
  return on_err;
}
}  // namespace ku
