// JSON dump (for people and offline tools) and a compact binary form (plan cache / replay).
#include <cstring>
#include <sstream>
#include <stdexcept>

#include "plan.h"

namespace fastb {

namespace {
void json_matrix(std::ostringstream& o, const Matrix& m) {
  o << "[";
  for (int i = 0; i < m.n; ++i) {
    o << (i ? "," : "") << "[";
    for (int j = 0; j < m.n; ++j) o << (j ? "," : "") << m.at(i, j);
    o << "]";
  }
  o << "]";
}
constexpr uint32_t kMagic = 0x46423230;  // "FB20"
constexpr uint32_t kVersion = 1;

struct Writer {
  std::vector<uint8_t> b;
  template <class T> void pod(const T& x) { const uint8_t* p = reinterpret_cast<const uint8_t*>(&x); b.insert(b.end(), p, p + sizeof(T)); }
  template <class T> void vec(const std::vector<T>& v) { pod<uint64_t>(v.size()); for (const T& x : v) pod(x); }
  void mat(const Matrix& m) { pod<int32_t>(m.n); vec(m.v); }
};
struct Reader {
  const std::vector<uint8_t>& b;
  size_t pos = 0;
  template <class T> T pod() {
    if (pos + sizeof(T) > b.size()) throw std::invalid_argument("plan_from_bytes: truncated blob");
    T x; std::memcpy(&x, &b[pos], sizeof(T)); pos += sizeof(T); return x;
  }
  template <class T> std::vector<T> vec() {
    uint64_t k = pod<uint64_t>();
    if (k > (b.size() - pos) / sizeof(T)) throw std::invalid_argument("plan_from_bytes: bad length");
    std::vector<T> v(k); for (auto& x : v) x = pod<T>(); return v;
  }
  Matrix mat() { Matrix m; m.n = pod<int32_t>(); m.v = vec<int64_t>(); if (m.v.size() != static_cast<size_t>(m.n) * m.n) throw std::invalid_argument("plan_from_bytes: bad matrix"); return m; }
};
}  // namespace

std::string plan_to_json(const Plan& p, bool include_ops) {
  std::ostringstream o;
  o << "{\"servers\":" << p.topo.servers << ",\"gpus\":" << p.topo.gpus << ",\"kind\":" << static_cast<int>(p.opt.kind)
    << ",\"transpose\":" << (p.opt.transpose ? "true" : "false") << ",\"matrix_hash\":\"" << std::hex << p.matrix_hash << std::dec
    << "\",\"num_stages\":" << p.num_stages << ",\"scale\":" << p.decomp.scale << ",\"line_sum\":" << p.decomp.line_sum << ",\"matrix\":";
  json_matrix(o, p.matrix);
  o << ",\"server_matrix\":";
  json_matrix(o, p.server_matrix);
  o << ",\"stages\":[";
  for (size_t k = 0; k < p.decomp.stages.size(); ++k) {
    const Stage& s = p.decomp.stages[k];
    o << (k ? "," : "") << "{\"weight\":" << s.weight << ",\"to\":[";
    for (size_t i = 0; i < s.to.size(); ++i) o << (i ? "," : "") << s.to[i];
    o << "]}";
  }
  o << "],\"buffers\":[";
  for (size_t r = 0; r < p.buffers.size(); ++r) {
    const RankBuffers& b = p.buffers[r];
    o << (r ? "," : "") << "{\"input\":" << b.input_units << ",\"output\":" << b.output_units << ",\"balance\":" << b.balance_units
      << ",\"rail\":" << b.rail_units << "}";
  }
  o << "]";
  if (include_ops) {
    o << ",\"ops\":[";
    for (size_t k = 0; k < p.ops.size(); ++k) {
      const Op& q = p.ops[k];
      o << (k ? "," : "") << "{\"phase\":" << static_cast<int>(q.phase) << ",\"stage\":" << q.stage << ",\"src\":" << q.src_rank
        << ",\"dst\":" << q.dst_rank << ",\"src_buf\":" << static_cast<int>(q.src_buf) << ",\"dst_buf\":" << static_cast<int>(q.dst_buf)
        << ",\"src_off\":" << q.src_off << ",\"dst_off\":" << q.dst_off << ",\"len\":" << q.len << ",\"origin\":" << q.origin
        << ",\"final\":" << q.final_dst << ",\"pair_off\":" << q.pair_off << "}";
    }
    o << "]";
  }
  o << "}";
  return o.str();
}

std::vector<uint8_t> plan_to_bytes(const Plan& p) {
  Writer w;
  w.pod(kMagic); w.pod(kVersion);
  w.pod<int32_t>(p.topo.servers); w.pod<int32_t>(p.topo.gpus);
  w.pod<int32_t>(static_cast<int>(p.opt.kind)); w.pod<int32_t>(static_cast<int>(p.opt.match));
  w.pod<int32_t>(static_cast<int>(p.opt.scale_policy)); w.pod<int64_t>(p.opt.scale); w.pod<int64_t>(p.opt.split_align);
  w.pod<int32_t>((p.opt.transpose ? 1 : 0) | (p.opt.balance_alpha_beta ? 2 : 0) | ((p.opt.only_rank + 1) << 8));
  w.mat(p.matrix); w.mat(p.server_matrix);
  w.mat(p.decomp.padded); w.mat(p.decomp.padding); w.pod(p.decomp.line_sum); w.pod(p.decomp.scale);
  w.pod<uint64_t>(p.decomp.stages.size());
  for (const Stage& s : p.decomp.stages) { w.pod(s.weight); w.vec(s.to); }
  w.pod(p.num_stages); w.vec(p.in_disp); w.vec(p.out_disp);
  w.pod<uint64_t>(p.buffers.size());
  for (const RankBuffers& b : p.buffers) { w.pod(b.input_units); w.pod(b.output_units); w.pod(b.balance_units); w.pod(b.rail_units); }
  w.pod<uint64_t>(p.ops.size());
  for (const Op& o : p.ops) {
    w.pod<uint8_t>(static_cast<uint8_t>(o.phase)); w.pod<uint8_t>(static_cast<uint8_t>(o.src_buf)); w.pod<uint8_t>(static_cast<uint8_t>(o.dst_buf));
    w.pod(o.stage); w.pod(o.src_rank); w.pod(o.dst_rank); w.pod(o.origin); w.pod(o.final_dst);
    w.pod(o.src_off); w.pod(o.dst_off); w.pod(o.len); w.pod(o.pair_off);
  }
  w.pod(p.matrix_hash);
  w.vec(p.rail_tail_start);  // appended after the first release of the format: absent in older blobs
  return w.b;
}

Plan plan_from_bytes(const std::vector<uint8_t>& blob) {
  Reader r{blob};
  if (r.pod<uint32_t>() != kMagic) throw std::invalid_argument("plan_from_bytes: not a plan blob");
  if (r.pod<uint32_t>() != kVersion) throw std::invalid_argument("plan_from_bytes: unsupported version");
  Plan p;
  p.topo.servers = r.pod<int32_t>(); p.topo.gpus = r.pod<int32_t>();
  p.opt.kind = static_cast<PlanKind>(r.pod<int32_t>()); p.opt.match = static_cast<MatchPolicy>(r.pod<int32_t>());
  p.opt.scale_policy = static_cast<ScalePolicy>(r.pod<int32_t>()); p.opt.scale = r.pod<int64_t>(); p.opt.split_align = r.pod<int64_t>();
  { const int32_t flags = r.pod<int32_t>(); p.opt.transpose = (flags & 1) != 0; p.opt.balance_alpha_beta = (flags & 2) != 0; p.opt.only_rank = (flags >> 8) - 1; }
  p.matrix = r.mat(); p.server_matrix = r.mat();
  p.decomp.padded = r.mat(); p.decomp.padding = r.mat(); p.decomp.line_sum = r.pod<int64_t>(); p.decomp.scale = r.pod<int64_t>();
  uint64_t ns = r.pod<uint64_t>();
  if (ns > blob.size()) throw std::invalid_argument("plan_from_bytes: bad stage count");
  p.decomp.stages.resize(ns);
  for (Stage& s : p.decomp.stages) { s.weight = r.pod<int64_t>(); s.to = r.vec<int>(); }
  p.num_stages = r.pod<int32_t>(); p.in_disp = r.vec<int64_t>(); p.out_disp = r.vec<int64_t>();
  uint64_t nb = r.pod<uint64_t>();
  if (nb > blob.size()) throw std::invalid_argument("plan_from_bytes: bad rank count");
  p.buffers.resize(nb);
  for (RankBuffers& b : p.buffers) { b.input_units = r.pod<int64_t>(); b.output_units = r.pod<int64_t>(); b.balance_units = r.pod<int64_t>(); b.rail_units = r.pod<int64_t>(); }
  uint64_t no = r.pod<uint64_t>();
  if (no > blob.size()) throw std::invalid_argument("plan_from_bytes: bad op count");
  p.ops.resize(no);
  for (Op& o : p.ops) {
    o.phase = static_cast<Phase>(r.pod<uint8_t>()); o.src_buf = static_cast<Buf>(r.pod<uint8_t>()); o.dst_buf = static_cast<Buf>(r.pod<uint8_t>());
    o.stage = r.pod<int32_t>(); o.src_rank = r.pod<int32_t>(); o.dst_rank = r.pod<int32_t>(); o.origin = r.pod<int32_t>(); o.final_dst = r.pod<int32_t>();
    o.src_off = r.pod<int64_t>(); o.dst_off = r.pod<int64_t>(); o.len = r.pod<int64_t>(); o.pair_off = r.pod<int64_t>();
  }
  p.matrix_hash = r.pod<uint64_t>();
  if (r.pos < blob.size()) {
    p.rail_tail_start = r.vec<int64_t>();
  } else {  // older blob: no tail recorded, which is right for every plan built without piece alignment
    for (const RankBuffers& b : p.buffers) p.rail_tail_start.push_back(b.rail_units);
  }
  return p;
}

}  // namespace fastb
