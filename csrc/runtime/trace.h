// Launch trace: device-timed events per kernel launch, kept in a bounded ring and
// fetched as JSON.  Counterpart of the reference's SysTraceGuard
// (spike/src/sys_trace.cpp:5-102) whose `nc_exec_running` start/stop device timestamps
// feed SpikeModel.benchmark(mode="device"); here every execute records a
// `kernel_exec` start/stop pair (CUDA events on the launch stream) plus, optionally,
// one pair per kernel launch of the plan.
#pragma once
#include <deque>
#include <mutex>
#include <string>

namespace spike {

struct TraceEvent {
  std::string name;        // "kernel_exec" or the kernel's symbol name
  std::string phase;       // "start" | "stop"
  long long tracking_id;   // one id per execute call
  double device_ns;        // nanoseconds on the device clock, relative to session start
  int core_id;
  std::string model;
};

class TraceSession {
 public:
  explicit TraceSession(int core_id = -1, size_t capacity = 65536);
  ~TraceSession();
  void stop();
  bool active() const { return active_; }
  int core_id() const { return core_id_; }
  void record(const TraceEvent& e);
  // returns and consumes the buffered events
  std::string fetch_events_json();
  void drain_events();
  long long next_tracking_id();

  static TraceSession* current();

 private:
  int core_id_;
  size_t capacity_;
  bool active_ = true;
  long long next_id_ = 0;
  std::deque<TraceEvent> events_;
  std::mutex mu_;
};

}  // namespace spike
