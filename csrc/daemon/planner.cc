#include "planner.h"

#include <algorithm>

#include "../common/protocol.h"

namespace mccs {

const TuneEntry* TuneTable::lookup(uint64_t bytes) const {
  for (const auto& e : entries)
    if (bytes <= e.max_bytes) return &e;
  return entries.empty() ? nullptr : &entries.back();
}

Planner::Planner() { load_defaults(false); }

TuneTable& Planner::table(int kind, int nranks) { return tables_[kind][nranks]; }
const TuneTable* Planner::find_table(int kind, int nranks) const {
  if (kind < 0 || kind >= kNumCollKinds || nranks < 1 || nranks > kMaxRanks) return nullptr;
  return &tables_[kind][nranks];
}

uint64_t Planner::message_bytes(const PlanInput& in) {
  // The whole message: what an all-gather produces, what a reduce-scatter consumes.
  if (in.kind == kAllGather) return in.count * (uint64_t)in.nranks;
  return send_units(in.kind, in.count, in.nranks) * (uint64_t)dtype_size(in.dtype);
}

int Planner::variant_from_name(const std::string& name) {
  if (name.empty() || name == "auto") return kAuto;
  for (int v = 1; v < kNumVariants; v++)
    if (name == variant_name(v)) return v;
  // Short aliases accepted in configuration files.
  if (name == "ring") return -2;   // resolved per collective kind by the caller
  if (name == "nvls") return -3;
  return -1;
}

void Planner::load_defaults(bool nvls) {
  std::unique_lock<std::shared_mutex> g(mu_);
  constexpr uint64_t KB = 1024, MB = 1024 * 1024;
  constexpr uint64_t kInf = ~0ull;
  for (int n = 1; n <= kMaxRanks; n++) {
    TuneTable& ar = table(kAllReduce, n);
    TuneTable& ag = table(kAllGather, n);
    TuneTable& rs = table(kReduceScatter, n);
    ar.entries.clear();
    ag.entries.clear();
    rs.entries.clear();
    if (n == 1) {
      ar.entries = {{1 * MB, kLocalCopy, 8, 512}, {kInf, kLocalCopy, 128, 512}};
      ag.entries = ar.entries;
      rs.entries = ar.entries;
      continue;
    }
    // Reduce-scatter has not been tuned on hardware: the rows follow the measured rows of
    // the kernels it shares its inner loop with (the reducing half of the two-shot exchange,
    // the in-switch reduction).
    if (n >= 4 && nvls)
      rs.entries = {{1 * MB, kRsDirect, 8, 512}, {32 * MB, kRsNvls, 8, 512}, {kInf, kRsNvls, 16, 512}};
    else
      rs.entries = {{1 * MB, kRsDirect, 8, 512}, {32 * MB, kRsDirect, 32, 512}, {kInf, kRsDirect, 64, 512}};
    // Rows measured on B200: eight ranks behind an NVSwitch for n >= 4, two ranks for
    // n <= 3, where the in-switch reduction moves no fewer bytes than a direct exchange
    // and measured slower. A tuning file replaces them per rank count.
    if (n <= 3) {
      ar.entries = {{2 * MB, kArOneShot, 32, 512},   {32 * MB, kArTwoShot, 64, 512},
                    {kInf, kArTwoShot, 128, 512}};
      ag.entries = {{128 * KB, kAgPull, 8, 512},     {2 * MB, kAgPush, 16, 512},
                    {64 * MB, kAgPush, 64, 512},     {kInf, kAgPush, 128, 512}};
    } else if (nvls) {
      ar.entries = {{256 * KB, kArNvlsOne, 4, 512},  {32 * MB, kArNvlsTwo, 8, 512},
                    {kInf, kArNvlsTwo, 16, 512}};
      ag.entries = {{128 * KB, kAgNvls, 2, 512},     {2 * MB, kAgPull, 32, 512},
                    {16 * MB, kAgPull, 64, 512},     {64 * MB, kAgPush, 32, 512},
                    {kInf, kAgPush, 128, 512}};
    } else {
      ar.entries = {{128 * KB, kArOneShot, 8, 512},  {4 * MB, kArTwoShot, 16, 512},
                    {64 * MB, kArTwoShot, 32, 512},  {kInf, kArTwoShot, 64, 512}};
      ag.entries = {{2 * MB, kAgPull, 32, 512},      {16 * MB, kAgPull, 64, 512},
                    {64 * MB, kAgPush, 32, 512},     {kInf, kAgPush, 128, 512}};
    }
  }
}

bool Planner::load_json(const Value& root, std::string* err) {
  // {"allreduce": {"8": [[max_bytes, "variant", ctas, threads], ...]}, "allgather": {...}}
  static const char* kind_names[kNumCollKinds] = {"allreduce", "allgather", "reducescatter"};
  for (int k = 0; k < kNumCollKinds; k++) {
    const Value& per_kind = root[kind_names[k]];
    for (const auto& kv : per_kind.fields()) {
      int n = atoi(kv.first.c_str());
      if (n < 1 || n > kMaxRanks) { if (err) *err = "bad rank count '" + kv.first + "'"; return false; }
      std::vector<TuneEntry> entries;
      for (const Value& row : kv.second.items()) {
        if (row.size() < 3) { if (err) *err = "tuning row needs [max_bytes, variant, ctas(, threads)]"; return false; }
        TuneEntry e;
        int64_t mb = row.at(0).as_int(-1);
        e.max_bytes = mb < 0 ? ~0ull : (uint64_t)mb;
        e.variant = variant_from_name(row.at(1).as_string());
        if (e.variant <= 0) { if (err) *err = "unknown variant '" + row.at(1).as_string() + "'"; return false; }
        e.ctas = (int)row.at(2).as_int(8);
        e.threads = (int)row.at(3).as_int(512);
        if (e.ctas < 1 || e.ctas > kMaxCtas || e.threads < 32 || e.threads > 512 || e.threads % 32) {
          if (err) *err = "tuning row out of range";
          return false;
        }
        entries.push_back(e);
      }
      if (entries.empty()) continue;
      std::unique_lock<std::shared_mutex> g(mu_);
      std::sort(entries.begin(), entries.end(),
                [](const TuneEntry& a, const TuneEntry& b) { return a.max_bytes < b.max_bytes; });
      entries.back().max_bytes = ~0ull;
      table(k, n).entries = entries;
    }
  }
  return true;
}

bool Planner::load_file(const std::string& path, std::string* err) {
  try {
    return load_json(parse_json(read_text_file(path)), err);
  } catch (const std::exception& e) {
    if (err) *err = e.what();
    return false;
  }
}

Value Planner::to_json() const {
  std::shared_lock<std::shared_mutex> g(mu_);
  static const char* kind_names[kNumCollKinds] = {"allreduce", "allgather", "reducescatter"};
  Value root = Value::object();
  for (int k = 0; k < kNumCollKinds; k++) {
    Value per_kind = Value::object();
    for (int n = 1; n <= kMaxRanks; n++) {
      Value rows = Value::array();
      for (const auto& e : tables_[k][n].entries) {
        Value row = Value::array();
        row.push(e.max_bytes == ~0ull ? Value((int64_t)-1) : Value((int64_t)e.max_bytes));
        row.push(variant_name(e.variant));
        row.push(e.ctas);
        row.push(e.threads);
        rows.push(row);
      }
      per_kind.set(std::to_string(n), rows);
    }
    root.set(kind_names[k], per_kind);
  }
  return root;
}

std::string Planner::infeasible(int variant, const PlanInput& in) {
  const bool is_ar = kind_reduces(in.kind);   // carries an element type and an operator
  switch (variant) {
    case kLocalCopy:
      return in.nranks == 1 ? "" : "local copy needs a single-rank communicator";
    case kArOneShot: case kArTwoShot: case kArRing: case kArNvlsOne: case kArNvlsTwo: case kArHybrid:
      if (in.kind != kAllReduce) return "all-reduce variant requested for another collective";
      break;
    case kAgPull: case kAgPush: case kAgNvls: case kAgRing:
      if (in.kind != kAllGather) return "all-gather variant requested for another collective";
      break;
    case kRsDirect: case kRsNvls:
      if (in.kind != kReduceScatter) return "reduce-scatter variant requested for another collective";
      break;
    default:
      return "unknown variant";
  }
  if (in.nranks == 1) return "single-rank communicator uses the local copy";
  if (in.host_staged && !variant_is_ring(variant)) return "host-staged transport only runs ring variants";
  if (!((in.carried_variants >> variant) & 1u)) return "a connection of this communicator cannot carry this variant";
  if (!variant_is_ring(variant) && !in.p2p_possible) return "no peer access between the devices";
  if (variant_is_nvls(variant)) {
    if (in.emulated) return "NVLS needs one device per rank";
    if (!in.nvls_possible) return "buffers are not multicast-mappable at equal offsets";
    if (!in.aligned16) return "NVLS needs 16-byte aligned buffers";
    if (is_ar) {
      if (in.dtype != kFloat32 && in.dtype != kFloat16 && in.dtype != kBfloat16)
        return "NVLS reduction supports f32/f16/bf16";
      if (in.op != kSum && in.op != kSumPostDiv) return "NVLS reduction supports sum";
    }
  }
  if ((variant == kArOneShot || variant == kArNvlsOne) && in.in_place)
    return "one-shot variants are out-of-place only";
  return "";
}

Plan Planner::plan(const PlanInput& in) const {
  constexpr uint64_t MB_ = 1024 * 1024;
  Plan p;
  p.bytes = message_bytes(in);
  if (in.nranks < 1 || in.nranks > kMaxRanks) { p.status = proto::kErrInvalidArgument; return p; }
  const bool is_ar = in.kind == kAllReduce;
  const bool is_rs = in.kind == kReduceScatter;
  std::shared_lock<std::shared_mutex> g(mu_);
  const TuneTable* t = find_table(in.kind, in.nranks);
  const TuneEntry* e = t ? t->lookup(p.bytes) : nullptr;

  // Candidate order: the requested variant, the table's pick, then safe fall-backs.
  std::vector<int> candidates;
  if (in.requested_variant > 0) candidates.push_back(in.requested_variant);
  if (e) candidates.push_back(e->variant);
  if (in.nranks == 1) candidates.push_back(kLocalCopy);
  if (is_rs) {
    candidates.push_back(kRsDirect);
  } else if (is_ar) {
    if (p.bytes <= 256 * 1024) candidates.push_back(kArOneShot);
    candidates.push_back(kArTwoShot);
    candidates.push_back(kArRing);
  } else {
    candidates.push_back(p.bytes <= 1024 * 1024 ? kAgPull : kAgPush);
    candidates.push_back(kAgPull);
    candidates.push_back(kAgRing);
  }
  int chosen = 0;
  for (int v : candidates) {
    std::string why = infeasible(v, in);
    if (why.empty()) { chosen = v; break; }
    if (p.note.empty() && (v == in.requested_variant || (e && v == e->variant)))
      p.note = std::string(variant_name(v)) + ": " + why;
  }
  if (!chosen) { p.status = proto::kErrUnsupported; return p; }
  p.variant = chosen;

  // Launch shape: the table row when it is for this variant, else a size-based guess.
  int ctas = 0, threads = 512;
  if (e && e->variant == chosen) { ctas = e->ctas; threads = e->threads; }
  if (!ctas) {
    const uint64_t MB = 1024 * 1024;
    ctas = p.bytes <= 256 * 1024 ? 4 : p.bytes <= 4 * MB ? 16 : p.bytes <= 64 * MB ? 32 : 64;
  }
  // The hybrid kernel runs two data paths side by side: the peer-copy part wants as many
  // CTAs as the plain two-shot exchange on top of the few that feed the switch.
  if (chosen == kArHybrid && !(e && e->variant == chosen)) ctas = p.bytes <= 4 * MB_ ? 24 : 72;
  if (variant_is_ring(chosen)) {
    ctas = in.ring_channels > 0 ? in.ring_channels : 1;
    // Small messages do not fill several channels: drop to one, then shrink the CTA,
    // as the reference does (plan.rs:602-635).
    const uint64_t per_rank = is_ar ? p.bytes : in.count;
    while (ctas > 1 && per_rank < (uint64_t)ctas * (uint64_t)threads * 64) ctas = 1;
    while (threads > 64 && per_rank < (uint64_t)ctas * (uint64_t)threads * 64) threads /= 2;
  }
  if (in.requested_ctas > 0) ctas = in.requested_ctas;
  if (in.cta_cap > 0 && ctas > in.cta_cap) ctas = in.cta_cap;
  if (variant_is_ring(chosen) && ctas > kMaxRingChannels) ctas = kMaxRingChannels;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas < 1) ctas = 1;
  // Never launch more CTAs than there are 16-byte packs per rank to move.
  const uint64_t packs = std::max<uint64_t>(1, p.bytes / 16 / (uint64_t)threads / (uint64_t)in.nranks);
  if (!variant_is_ring(chosen) && (uint64_t)ctas > packs) ctas = (int)packs;
  p.dims.ctas = ctas;
  p.dims.threads = threads;
  p.needs_mc_send = chosen == kArNvlsOne || chosen == kArNvlsTwo || chosen == kArHybrid || chosen == kRsNvls;
  p.needs_mc_recv = chosen == kArNvlsTwo || chosen == kAgNvls || chosen == kArHybrid;
  return p;
}

}  // namespace mccs
