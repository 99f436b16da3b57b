// Membership master of the fault-tolerant collective layer, as a native service.
//
// The reference delegates this role to the master process of the PCCL library behind its ftccl wrapper (reference:
// ftccl/include/ftccl.h:198-229 — CreateMaster / RunMaster / InterruptMaster; src/main.cpp:266-320, 401-425 — how the
// trainer votes on topology updates and waits for the world size).
//
// Peers hold one TCP connection to the master and exchange newline-terminated JSON objects with it:
//
//   {"op":"connect","peer_group":g,"ip":"a.b.c.d"}          -> {"ok":true,"uid":u}
//   {"op":"heartbeat"}                                      -> {"epoch":e,"pending":p,"world":w,"ok":known}
//   {"op":"pending"}                                        -> {"ok":true,"pending":p}
//   {"op":"vote","free_port":n,"min_world":m,"timeout":s}   -> the new topology once every live accepted peer (and
//                                                              every peer waiting for admission) has voted:
//        {"ok":true,"epoch":e,"world":w,"ranks":{"uid":rank,..},"store":{"ip":..,"port":..},"groups":{"uid":g,..}}
//   {"op":"gate","step":s,"epoch":e,"world":w,"timeout":s}  -> {"ok":true,"aligned":true|false,...}: host-side step
//                                                              barrier; not aligned = membership differs, re-vote
//   {"op":"leave"}                                          -> {"ok":true}
//
// A peer that stops sending anything for `heartbeat_timeout` seconds is evicted, which also unblocks votes and
// gates that were waiting for it.  The role corresponds to the master process of the reference's fault-tolerant
// communication library (ftccl/include/ftccl.h:223-227: CreateMaster / RunMaster / Interrupt / AwaitTermination);
// the protocol is this project's own.
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "json_min.h"

namespace {

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct PeerRec {
  int uid = 0;
  int group = 0;
  std::string ip;
  double last_seen = 0;
  bool accepted = false;
  bool has_vote = false;
  int vote_port = 0;
  int vote_min_world = 1;
  bool has_gate = false;
  long long gate_step = -1;
};

struct Topology {
  long long round = 0;
  int epoch = 0;
  std::vector<std::pair<int, int>> ranks;   // uid -> rank
  std::vector<std::pair<int, int>> groups;  // uid -> peer group
  std::string store_ip;
  int store_port = 0;
  bool has(int uid) const {
    for (const auto& r : ranks)
      if (r.first == uid) return true;
    return false;
  }
};

double num(const fbam::JsonValue& v, const char* key, double fallback) {
  const fbam::JsonValue* f = v.find(key);
  return (f != nullptr && f->kind == fbam::JsonValue::Number) ? f->number : fallback;
}
std::string str(const fbam::JsonValue& v, const char* key, const std::string& fallback) {
  const fbam::JsonValue* f = v.find(key);
  return (f != nullptr && f->kind == fbam::JsonValue::String) ? f->str : fallback;
}

class Master {
 public:
  Master(const char* ip, int port, double heartbeat_timeout) : hb_timeout_(heartbeat_timeout) {
    fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd_ < 0) return;
    int one = 1;
    setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(static_cast<uint16_t>(port));
    if (inet_pton(AF_INET, ip, &addr.sin_addr) != 1 || bind(fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 ||
        listen(fd_, 64) != 0) {
      ::close(fd_);
      fd_ = -1;
      return;
    }
    socklen_t len = sizeof(addr);
    getsockname(fd_, reinterpret_cast<sockaddr*>(&addr), &len);
    port_ = ntohs(addr.sin_port);
    acceptor_ = std::thread([this] { accept_loop(); });
  }

  ~Master() {
    stop_ = true;
    cv_.notify_all();
    if (acceptor_.joinable()) acceptor_.join();
    // connection threads notice stop_ within one poll interval
    for (int i = 0; i < 100 && live_threads_.load() > 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(20));
    if (fd_ >= 0) ::close(fd_);
  }

  bool ok() const { return fd_ >= 0; }
  int port() const { return port_; }

  std::string snapshot() {
    std::lock_guard<std::mutex> lock(mu_);
    std::string acc, pen;
    for (const auto& kv : peers_) {
      std::string& dst = kv.second.accepted ? acc : pen;
      if (!dst.empty()) dst += ",";
      dst += std::to_string(kv.first);
    }
    return "{\"epoch\":" + std::to_string(epoch_) + ",\"accepted\":[" + acc + "],\"pending\":[" + pen + "]}";
  }

 private:
  int fd_ = -1, port_ = 0;
  double hb_timeout_;
  std::atomic<bool> stop_{false};
  std::atomic<int> live_threads_{0};
  std::thread acceptor_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::map<int, PeerRec> peers_;
  int next_uid_ = 1;
  int epoch_ = 0;
  Topology topo_;

  bool alive(const PeerRec& p) const { return now_s() - p.last_seen <= hb_timeout_; }

  void evict_silent(int except_uid) {  // with mu_ held
    bool any = false;
    for (auto it = peers_.begin(); it != peers_.end();) {
      if (it->first != except_uid && !alive(it->second)) {
        it = peers_.erase(it);
        any = true;
      } else {
        ++it;
      }
    }
    if (any) cv_.notify_all();
  }

  // With mu_ held: completes the voting round if every live accepted peer and every waiting peer has voted.
  void try_complete_round() {
    std::vector<PeerRec*> members;
    bool any_vote = false, any_accepted = false;
    for (auto& kv : peers_) {
      PeerRec& p = kv.second;
      if (!alive(p)) continue;
      any_vote = any_vote || p.has_vote;
      any_accepted = any_accepted || p.accepted;
      if (p.accepted || p.has_vote) members.push_back(&p);
    }
    if (!any_vote) return;
    int min_world = 1;
    for (PeerRec* p : members) {
      if (!p->has_vote) return;  // an accepted peer has not voted yet
      if (p->vote_min_world > min_world) min_world = p->vote_min_world;
    }
    if (static_cast<int>(members.size()) < min_world) return;  // keep waiting for more peers
    (void)any_accepted;
    ++epoch_;
    Topology t;
    t.round = topo_.round + 1;
    t.epoch = epoch_;
    t.store_ip = members.front()->ip;
    t.store_port = members.front()->vote_port;
    int rank = 0;
    for (PeerRec* p : members) {  // std::map iteration order = ascending uid
      t.ranks.emplace_back(p->uid, rank++);
      t.groups.emplace_back(p->uid, p->group);
      p->accepted = true;
      p->has_vote = false;   // gate marks are kept: members that re-voted from inside a step's gate go straight on
                             // to that step's collective, and a joiner's gate for the same step must see them
    }
    topo_ = t;
    cv_.notify_all();
  }

  static std::string topology_json(const Topology& t) {
    std::string ranks, groups;
    for (const auto& r : t.ranks) {
      if (!ranks.empty()) ranks += ",";
      ranks += "\"" + std::to_string(r.first) + "\":" + std::to_string(r.second);
    }
    for (const auto& g : t.groups) {
      if (!groups.empty()) groups += ",";
      groups += "\"" + std::to_string(g.first) + "\":" + std::to_string(g.second);
    }
    return "{\"ok\":true,\"epoch\":" + std::to_string(t.epoch) + ",\"world\":" + std::to_string(t.ranks.size()) +
           ",\"round\":" + std::to_string(t.round) + ",\"ranks\":{" + ranks + "},\"store\":{\"ip\":\"" + t.store_ip +
           "\",\"port\":" + std::to_string(t.store_port) + "},\"groups\":{" + groups + "}}";
  }

  void accept_loop() {
    while (!stop_) {
      pollfd p{fd_, POLLIN, 0};
      const int r = ::poll(&p, 1, 200);
      if (r <= 0) {
        std::lock_guard<std::mutex> lock(mu_);
        evict_silent(-1);
        continue;
      }
      sockaddr_in peer{};
      socklen_t len = sizeof(peer);
      const int c = ::accept(fd_, reinterpret_cast<sockaddr*>(&peer), &len);
      if (c < 0) continue;
      int one = 1;
      setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      char ipbuf[64] = {0};
      inet_ntop(AF_INET, &peer.sin_addr, ipbuf, sizeof(ipbuf));
      ++live_threads_;
      std::thread([this, c, ip = std::string(ipbuf)] {
        serve(c, ip);
        ::close(c);
        --live_threads_;
      }).detach();
    }
  }

  // Reads one line; false on disconnect or shutdown.
  bool read_line(int c, std::string& carry, std::string& line) {
    while (!stop_) {
      const size_t nl = carry.find('\n');
      if (nl != std::string::npos) {
        line = carry.substr(0, nl);
        carry.erase(0, nl + 1);
        return true;
      }
      pollfd p{c, POLLIN, 0};
      const int r = ::poll(&p, 1, 200);
      if (r < 0) return false;
      if (r == 0) continue;
      char buf[4096];
      const ssize_t n = ::recv(c, buf, sizeof(buf), 0);
      if (n <= 0) return false;
      carry.append(buf, static_cast<size_t>(n));
    }
    return false;
  }

  static bool send_line(int c, const std::string& s) {
    std::string out = s + "\n";
    size_t off = 0;
    while (off < out.size()) {
      const ssize_t n = ::send(c, out.data() + off, out.size() - off, MSG_NOSIGNAL);
      if (n <= 0) return false;
      off += static_cast<size_t>(n);
    }
    return true;
  }

  void serve(int c, const std::string& remote_ip) {
    std::string carry, line;
    int uid = -1;
    while (read_line(c, carry, line)) {
      fbam::JsonValue msg;
      try {
        msg = fbam::JsonParser(line).parse();
      } catch (const std::exception&) {
        return;
      }
      const std::string op = str(msg, "op", "");
      {
        std::lock_guard<std::mutex> lock(mu_);
        auto it = peers_.find(uid);
        if (it != peers_.end()) it->second.last_seen = now_s();
      }
      std::string reply;
      if (op == "connect") {
        std::lock_guard<std::mutex> lock(mu_);
        uid = next_uid_++;
        PeerRec p;
        p.uid = uid;
        p.group = static_cast<int>(num(msg, "peer_group", 0));
        p.ip = str(msg, "ip", remote_ip);
        p.last_seen = now_s();
        peers_[uid] = p;
        cv_.notify_all();
        reply = "{\"ok\":true,\"uid\":" + std::to_string(uid) + "}";
      } else if (op == "heartbeat") {
        std::lock_guard<std::mutex> lock(mu_);
        int pending = 0, world = 0;
        for (const auto& kv : peers_) {
          if (!kv.second.accepted) ++pending;
          else if (alive(kv.second)) ++world;
        }
        reply = "{\"epoch\":" + std::to_string(epoch_) + ",\"pending\":" + std::to_string(pending) + ",\"world\":" +
                std::to_string(world) + ",\"ok\":" + (peers_.count(uid) ? "true" : "false") + "}";
      } else if (op == "pending") {
        std::lock_guard<std::mutex> lock(mu_);
        int pending = 0;
        for (const auto& kv : peers_)
          if (!kv.second.accepted && alive(kv.second)) ++pending;
        reply = "{\"ok\":true,\"pending\":" + std::to_string(pending) + "}";
      } else if (op == "vote") {
        reply = vote(uid, msg);
      } else if (op == "gate") {
        reply = gate(uid, msg);
      } else if (op == "leave") {
        {
          std::lock_guard<std::mutex> lock(mu_);
          peers_.erase(uid);
          cv_.notify_all();
        }
        send_line(c, "{\"ok\":true}");
        return;
      } else {
        reply = "{\"ok\":false,\"error\":\"unknown op\"}";
      }
      if (!send_line(c, reply)) return;
    }
  }

  std::string vote(int uid, const fbam::JsonValue& msg) {
    const double deadline = now_s() + num(msg, "timeout", 30.0);
    std::unique_lock<std::mutex> lock(mu_);
    auto it = peers_.find(uid);
    if (it == peers_.end()) return "{\"ok\":false,\"error\":\"evicted\"}";
    const long long start_round = topo_.round;
    it->second.has_vote = true;
    it->second.vote_port = static_cast<int>(num(msg, "free_port", 0));
    it->second.vote_min_world = static_cast<int>(num(msg, "min_world", 1));
    try_complete_round();
    while (topo_.round == start_round && !stop_) {
      const double remaining = deadline - now_s();
      if (remaining <= 0) break;
      cv_.wait_for(lock, std::chrono::duration<double>(remaining < 0.2 ? remaining : 0.2));
      auto me = peers_.find(uid);
      if (me != peers_.end()) me->second.last_seen = now_s();
      evict_silent(uid);  // a dead accepted peer must not block the round
      if (topo_.round == start_round) try_complete_round();
    }
    if (topo_.round != start_round && topo_.has(uid)) return topology_json(topo_);
    auto me = peers_.find(uid);
    if (me != peers_.end()) me->second.has_vote = false;
    return "{\"ok\":false,\"error\":\"timeout\"}";
  }

  std::string gate(int uid, const fbam::JsonValue& msg) {
    const long long step = static_cast<long long>(num(msg, "step", -1));
    const double deadline = now_s() + num(msg, "timeout", 30.0);
    std::unique_lock<std::mutex> lock(mu_);
    auto it = peers_.find(uid);
    if (it == peers_.end()) return "{\"ok\":false,\"error\":\"evicted\"}";
    it->second.has_gate = true;
    it->second.gate_step = step;
    cv_.notify_all();
    while (!stop_) {
      int accepted = 0, pending = 0;
      bool all_here = true;
      for (const auto& kv : peers_) {
        const PeerRec& p = kv.second;
        if (!(alive(p) || p.uid == uid)) continue;
        if (!p.accepted) { ++pending; continue; }
        ++accepted;
        if (!p.has_gate || p.gate_step < step) all_here = false;
      }
      const bool changed = pending > 0 || static_cast<int>(num(msg, "epoch", epoch_)) != epoch_ ||
                           accepted != static_cast<int>(num(msg, "world", accepted));
      const std::string tail = ",\"world\":" + std::to_string(accepted) + ",\"pending\":" + std::to_string(pending) +
                               ",\"epoch\":" + std::to_string(epoch_) + "}";
      if (changed) return "{\"ok\":true,\"aligned\":false" + tail;
      if (all_here) return "{\"ok\":true,\"aligned\":true" + tail;
      const double remaining = deadline - now_s();
      if (remaining <= 0) return "{\"ok\":true,\"aligned\":false,\"timeout\":true" + tail;
      cv_.wait_for(lock, std::chrono::duration<double>(remaining < 0.05 ? remaining : 0.05));
      auto me = peers_.find(uid);
      if (me == peers_.end()) return "{\"ok\":false,\"error\":\"evicted\"}";
      me->second.last_seen = now_s();
      evict_silent(uid);
    }
    return "{\"ok\":false,\"error\":\"stopped\"}";
  }
};

}  // namespace

extern "C" {

// Starts a master on ip:port (port 0 = any free port).  Returns a handle or null; *out_port receives the port.
void* fbam_master_start(const char* ip, int port, double heartbeat_timeout_s, int* out_port) {
  Master* m = new Master(ip, port, heartbeat_timeout_s);
  if (!m->ok()) {
    delete m;
    return nullptr;
  }
  if (out_port != nullptr) *out_port = m->port();
  return m;
}

// Stops accepting, wakes every waiting request and closes the listener.
void fbam_master_stop(void* h) { delete static_cast<Master*>(h); }

// {"epoch":e,"accepted":[uids],"pending":[uids]} into buf; returns the length needed (excluding the terminator).
int fbam_master_snapshot(void* h, char* buf, int cap) {
  const std::string s = static_cast<Master*>(h)->snapshot();
  if (buf != nullptr && cap > 0) {
    const size_t n = s.size() < static_cast<size_t>(cap - 1) ? s.size() : static_cast<size_t>(cap - 1);
    memcpy(buf, s.data(), n);
    buf[n] = 0;
  }
  return static_cast<int>(s.size());
}

}  // extern "C"
