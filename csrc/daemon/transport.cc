#include "transport.h"

#include <map>

namespace mccs {

namespace {

class NvlsTransport : public Transport {
 public:
  TransportKind kind() const override { return kTransportNvls; }
  const char* name() const override { return "nvls"; }
  bool can_connect(const TransportEnv& env, int s, int r) const override {
    // Multicast objects join distinct devices; both ends must be able to take part, and the
    // unicast halves of the kernels (tails, flags) need peer access as well.
    return env.nvls_enabled && s != r && env.multicast && env.multicast(s) && env.multicast(r) && env.peer_access &&
           env.peer_access(s, r) && env.peer_access(r, s);
  }
  bool carries(int variant) const override { return variant > kAuto && variant < kNumVariants; }
  bool scratch_in_host_memory() const override { return false; }
};

class NvlinkP2PTransport : public Transport {
 public:
  TransportKind kind() const override { return kTransportNvlinkP2P; }
  const char* name() const override { return "nvlink_p2p"; }
  bool can_connect(const TransportEnv& env, int s, int r) const override {
    // Two ranks on one device address the same memory anyway.
    return s == r || (env.peer_access && env.peer_access(s, r) && env.peer_access(r, s));
  }
  bool carries(int variant) const override { return variant > kAuto && variant < kNumVariants && !variant_is_nvls(variant); }
  bool scratch_in_host_memory() const override { return false; }
};

class HostStagedTransport : public Transport {
 public:
  TransportKind kind() const override { return kTransportHostStaged; }
  const char* name() const override { return "host_staged"; }
  bool can_connect(const TransportEnv&, int, int) const override { return true; }   // pinned host memory is visible to every GPU
  bool carries(int variant) const override { return variant_is_ring(variant); }
  bool scratch_in_host_memory() const override { return true; }
};

}  // namespace

TransportCatalog::TransportCatalog(const std::string& mode) {
  if (mode != "host_staged") {
    list_.emplace_back(new NvlsTransport());
    list_.emplace_back(new NvlinkP2PTransport());
  }
  if (mode != "nvlink") list_.emplace_back(new HostStagedTransport());
}

const Transport* TransportCatalog::select(const TransportEnv& env, int send_dev, int recv_dev) const {
  for (const auto& t : list_)
    if (t->can_connect(env, send_dev, recv_dev)) return t.get();
  return nullptr;
}

ConnectionTable connect_all(const TransportCatalog& catalog, const TransportEnv& env, const std::vector<int>& devices) {
  ConnectionTable t;
  t.nranks = (int)devices.size();
  for (int a = 0; a < t.nranks; a++)
    for (int b = 0; b < t.nranks; b++) {
      if (a == b) continue;
      t.conn[a][b] = catalog.select(env, devices[(size_t)a], devices[(size_t)b]);
      if (!t.conn[a][b] && t.unconnected_from < 0) { t.unconnected_from = a; t.unconnected_to = b; }
    }
  return t;
}

bool ConnectionTable::any(TransportKind k) const {
  for (int a = 0; a < nranks; a++)
    for (int b = 0; b < nranks; b++)
      if (a != b && conn[a][b] && conn[a][b]->kind() == k) return true;
  return false;
}

bool ConnectionTable::all(TransportKind k) const {
  for (int a = 0; a < nranks; a++)
    for (int b = 0; b < nranks; b++)
      if (a != b && (!conn[a][b] || conn[a][b]->kind() != k)) return false;
  return true;
}

bool ConnectionTable::carries(int variant) const {
  for (int a = 0; a < nranks; a++)
    for (int b = 0; b < nranks; b++)
      if (a != b && (!conn[a][b] || !conn[a][b]->carries(variant))) return false;
  return true;
}

bool ConnectionTable::scratch_in_host_memory() const {
  for (int a = 0; a < nranks; a++)
    for (int b = 0; b < nranks; b++)
      if (a != b && conn[a][b] && conn[a][b]->scratch_in_host_memory()) return true;
  return false;
}

uint32_t ConnectionTable::carried_variants() const {
  uint32_t m = 0;
  for (int v = kAuto + 1; v < kNumVariants; v++)
    if (carries(v)) m |= 1u << v;
  return m;
}

std::string ConnectionTable::describe() const {
  std::map<std::string, int> n;
  for (int a = 0; a < nranks; a++)
    for (int b = 0; b < nranks; b++)
      if (a != b) n[conn[a][b] ? conn[a][b]->name() : "unconnected"]++;
  if (n.empty()) return "no connections";
  if (n.size() == 1) return n.begin()->first;
  std::string s;
  for (auto& kv : n) s += (s.empty() ? "" : ", ") + kv.first + " x" + std::to_string(kv.second);
  return s;
}

}  // namespace mccs
