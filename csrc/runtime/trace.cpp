#include "trace.h"

#include <sstream>

#include "error.h"
#include "json.h"

namespace spike {

static TraceSession* g_current = nullptr;
static std::mutex g_mu;

TraceSession::TraceSession(int core_id, size_t capacity) : core_id_(core_id), capacity_(capacity) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_current) throw SpikeError("a system trace session is already active");
  g_current = this;
}

TraceSession::~TraceSession() { stop(); }

void TraceSession::stop() {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_current == this) g_current = nullptr;
  active_ = false;
}

TraceSession* TraceSession::current() {
  std::lock_guard<std::mutex> lock(g_mu);
  return g_current;
}

void TraceSession::record(const TraceEvent& e) {
  std::lock_guard<std::mutex> lock(mu_);
  if (!active_) return;
  if (core_id_ >= 0 && e.core_id != core_id_) return;
  if (events_.size() >= capacity_) events_.pop_front();
  events_.push_back(e);
}

long long TraceSession::next_tracking_id() {
  std::lock_guard<std::mutex> lock(mu_);
  return next_id_++;
}

std::string TraceSession::fetch_events_json() {
  std::deque<TraceEvent> taken;
  {
    std::lock_guard<std::mutex> lock(mu_);
    taken.swap(events_);
  }
  std::ostringstream os;
  os.precision(17);
  os << "{\"events\": [";
  bool first = true;
  for (const auto& e : taken) {
    if (!first) os << ", ";
    first = false;
    os << "{\"event_type\": " << Json::quote(e.name) << ", \"phase\": " << Json::quote(e.phase)
       << ", \"tracking_id\": " << e.tracking_id << ", \"device_timestamp_ns\": " << e.device_ns
       << ", \"core_id\": " << e.core_id << ", \"model\": " << Json::quote(e.model) << "}";
  }
  os << "]}";
  return os.str();
}

void TraceSession::drain_events() {
  std::lock_guard<std::mutex> lock(mu_);
  events_.clear();
}

}  // namespace spike
