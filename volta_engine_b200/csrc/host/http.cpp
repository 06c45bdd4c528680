// Single-threaded epoll HTTP/1.1 front end with keep-alive, chunked / SSE streaming and per-connection
// non-blocking outbound queues. Parsed requests are handed to the embedding runtime through a queue
// (vh_http_next); responses and stream chunks come back through thread-safe calls that only enqueue bytes
// and wake the epoll thread. Same responsibilities as the reference's server core
// (src/server/http.cpp, src/server/server.cpp:128-162,229; behaviour notes docs/server.md:10-74):
// idle timeout, outbound-queue overflow drops the connection, client-gone detection.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace vh {

static double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct Conn {
  int fd = -1;
  uint64_t id = 0;
  std::string in;            // unparsed input
  std::string out;           // bytes waiting for the socket
  bool close_after_flush = false;
  bool busy = false;         // a request of this connection is being handled
  bool streaming = false;
  bool keep_alive = true;
  double last_io = 0;
};

struct PendingReq {
  uint64_t conn;
  std::string blob;          // method \n target \n header lines \n\n body
};

struct Server {
  int lfd = -1, ep = -1, evfd = -1, port = 0;
  std::thread th;
  std::atomic<bool> stop{false};
  std::mutex mu;             // guards conns' out / flags and the queues
  std::condition_variable cv;
  std::map<uint64_t, Conn*> conns;
  std::map<int, uint64_t> by_fd;
  std::deque<PendingReq> reqs;
  uint64_t next_id = 1;
  size_t max_body = 64u << 20, max_out = 64u << 20;
  double idle_timeout = 300.0;
  std::atomic<uint64_t> n_requests{0}, n_dropped{0};

  void wake() {
    uint64_t one = 1;
    ssize_t r = write(evfd, &one, 8);
    (void)r;
  }
  void mod(Conn* c) {
    epoll_event ev{};
    ev.events = EPOLLIN | (c->out.empty() ? 0 : EPOLLOUT) | EPOLLRDHUP;
    ev.data.fd = c->fd;
    epoll_ctl(ep, EPOLL_CTL_MOD, c->fd, &ev);
  }
  void drop(Conn* c) {
    epoll_ctl(ep, EPOLL_CTL_DEL, c->fd, nullptr);
    close(c->fd);
    by_fd.erase(c->fd);
    conns.erase(c->id);
    delete c;
  }
  // Tries to cut one complete request out of c->in. Returns true when a request was queued.
  bool parse(Conn* c) {
    size_t he = c->in.find("\r\n\r\n");
    if (he == std::string::npos) {
      if (c->in.size() > 65536) { c->close_after_flush = true; reply_simple(c, 431, "header too large"); }
      return false;
    }
    size_t clen = 0;
    bool keep = true;
    {
      // case-insensitive scan of the header block
      std::string hdr = c->in.substr(0, he);
      std::string low = hdr;
      for (auto& ch : low) ch = (char)tolower((unsigned char)ch);
      size_t p = low.find("\r\ncontent-length:");
      if (p != std::string::npos) clen = (size_t)strtoull(hdr.c_str() + p + 17, nullptr, 10);
      if (low.find("\r\nconnection: close") != std::string::npos) keep = false;
      if (low.find("\r\ntransfer-encoding: chunked") != std::string::npos) { reply_simple(c, 411, "length required"); c->close_after_flush = true; return false; }
      if (low.compare(0, 5, "get /") != 0 && low.compare(0, 6, "post /") != 0 && low.compare(0, 9, "options /") != 0 &&
          low.compare(0, 6, "head /") != 0 && low.compare(0, 8, "delete /") != 0) {
        reply_simple(c, 400, "bad request");
        c->close_after_flush = true;
        return false;
      }
    }
    if (clen > max_body) { reply_simple(c, 413, "body too large"); c->close_after_flush = true; return false; }
    if (c->in.size() < he + 4 + clen) return false;
    std::string head = c->in.substr(0, he), body = c->in.substr(he + 4, clen);
    c->in.erase(0, he + 4 + clen);
    // request line
    size_t le = head.find("\r\n");
    std::string line = head.substr(0, le), rest = le == std::string::npos ? "" : head.substr(le + 2);
    size_t s1 = line.find(' '), s2 = line.rfind(' ');
    if (s1 == std::string::npos || s2 <= s1) { reply_simple(c, 400, "bad request line"); c->close_after_flush = true; return false; }
    PendingReq r;
    r.conn = c->id;
    r.blob = line.substr(0, s1) + "\n" + line.substr(s1 + 1, s2 - s1 - 1) + "\n";
    for (size_t i = 0; i < rest.size();) {
      size_t e = rest.find("\r\n", i);
      if (e == std::string::npos) e = rest.size();
      r.blob += rest.substr(i, e - i) + "\n";
      i = e + 2;
    }
    r.blob += "\n";
    r.blob += body;
    c->busy = true;
    c->keep_alive = keep;
    reqs.push_back(std::move(r));
    n_requests++;
    cv.notify_one();
    return true;
  }
  void reply_simple(Conn* c, int code, const char* msg) {
    char buf[256];
    int n = snprintf(buf, sizeof buf, "HTTP/1.1 %d Error\r\nContent-Type: text/plain\r\nContent-Length: %zu\r\nConnection: close\r\n\r\n%s",
                     code, strlen(msg), msg);
    c->out.append(buf, (size_t)n);
    mod(c);
  }
  void flush(Conn* c) {
    while (!c->out.empty()) {
      ssize_t n = send(c->fd, c->out.data(), c->out.size(), MSG_NOSIGNAL);
      if (n > 0) { c->out.erase(0, (size_t)n); c->last_io = now_s(); }
      else if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) break;
      else { drop(c); return; }
    }
    if (c->out.empty() && c->close_after_flush) { drop(c); return; }
    mod(c);
  }
  void loop() {
    std::vector<epoll_event> evs(256);
    double last_sweep = now_s();
    while (!stop.load()) {
      int n = epoll_wait(ep, evs.data(), (int)evs.size(), 500);
      std::unique_lock<std::mutex> lk(mu);
      for (int i = 0; i < n; ++i) {
        int fd = evs[i].data.fd;
        if (fd == evfd) {
          uint64_t v;
          ssize_t r = read(evfd, &v, 8);
          (void)r;
          // flush every connection that has queued output (cheap: few connections)
          std::vector<Conn*> todo;
          for (auto& kv : conns) if (!kv.second->out.empty() || kv.second->close_after_flush) todo.push_back(kv.second);
          for (auto* c : todo) if (conns.count(c->id)) flush(c);
          continue;
        }
        if (fd == lfd) {
          for (;;) {
            int cfd = accept4(lfd, nullptr, nullptr, SOCK_NONBLOCK);
            if (cfd < 0) break;
            int one = 1;
            setsockopt(cfd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
            auto* c = new Conn();
            c->fd = cfd;
            c->id = next_id++;
            c->last_io = now_s();
            conns[c->id] = c;
            by_fd[cfd] = c->id;
            epoll_event ev{};
            ev.events = EPOLLIN | EPOLLRDHUP;
            ev.data.fd = cfd;
            epoll_ctl(ep, EPOLL_CTL_ADD, cfd, &ev);
          }
          continue;
        }
        auto it = by_fd.find(fd);
        if (it == by_fd.end()) continue;
        Conn* c = conns[it->second];
        if (evs[i].events & (EPOLLHUP | EPOLLERR)) { drop(c); continue; }
        if (evs[i].events & EPOLLIN) {
          char buf[65536];
          bool gone = false;
          for (;;) {
            ssize_t r = recv(fd, buf, sizeof buf, 0);
            if (r > 0) { c->in.append(buf, (size_t)r); c->last_io = now_s(); if (c->in.size() > max_body + 65536) { gone = true; break; } }
            else if (r == 0) { gone = true; break; }
            else if (errno == EAGAIN || errno == EWOULDBLOCK) break;
            else { gone = true; break; }
          }
          if (gone) { drop(c); continue; }
          if (!c->busy) parse(c);
        }
        if (conns.count(it->second) && (evs[i].events & EPOLLOUT)) flush(c);
        else if ((evs[i].events & EPOLLRDHUP) && conns.count(it->second) && !c->busy) drop(c);
      }
      double t = now_s();
      if (t - last_sweep > 5.0) {
        last_sweep = t;
        std::vector<Conn*> idle;
        for (auto& kv : conns) if (!kv.second->busy && t - kv.second->last_io > idle_timeout) idle.push_back(kv.second);
        for (auto* c : idle) drop(c);
      }
    }
  }
  // enqueue bytes for a connection (any thread). Returns 0, or -1 when the connection is gone / dropped.
  int enqueue(uint64_t id, const char* data, size_t n, bool finish_request, bool close_conn) {
    std::lock_guard<std::mutex> lk(mu);
    auto it = conns.find(id);
    if (it == conns.end()) return -1;
    Conn* c = it->second;
    if (c->out.size() + n > max_out) {   // slow reader: drop instead of buffering without bound
      n_dropped++;
      c->close_after_flush = true;
      c->out.clear();
      wake();
      return -1;
    }
    c->out.append(data, n);
    if (finish_request) {
      c->busy = false;
      c->streaming = false;
      if (close_conn || !c->keep_alive) c->close_after_flush = true;
      else if (!c->in.empty()) parse(c);   // pipelined request already buffered
    }
    wake();
    return 0;
  }
};

}  // namespace vh

using namespace vh;

extern "C" {

void* vh_http_start(const char* host, int port, int idle_timeout_s) {
  auto* s = new Server();
  s->lfd = socket(AF_INET, SOCK_STREAM | SOCK_NONBLOCK, 0);
  if (s->lfd < 0) { delete s; return nullptr; }
  int one = 1;
  setsockopt(s->lfd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)port);
  if (!host || !*host || inet_pton(AF_INET, host, &a.sin_addr) != 1) a.sin_addr.s_addr = htonl(INADDR_ANY);
  if (bind(s->lfd, (sockaddr*)&a, sizeof a) != 0 || listen(s->lfd, 512) != 0) { close(s->lfd); delete s; return nullptr; }
  socklen_t al = sizeof a;
  getsockname(s->lfd, (sockaddr*)&a, &al);
  s->port = ntohs(a.sin_port);
  if (idle_timeout_s > 0) s->idle_timeout = idle_timeout_s;
  s->ep = epoll_create1(0);
  s->evfd = eventfd(0, EFD_NONBLOCK);
  epoll_event ev{};
  ev.events = EPOLLIN;
  ev.data.fd = s->lfd;
  epoll_ctl(s->ep, EPOLL_CTL_ADD, s->lfd, &ev);
  ev.data.fd = s->evfd;
  epoll_ctl(s->ep, EPOLL_CTL_ADD, s->evfd, &ev);
  s->th = std::thread([s] { s->loop(); });
  return s;
}

int vh_http_port(void* h) { return ((Server*)h)->port; }

void vh_http_stop(void* h) {
  auto* s = (Server*)h;
  s->stop = true;
  s->wake();
  if (s->th.joinable()) s->th.join();
  {
    std::lock_guard<std::mutex> lk(s->mu);
    for (auto& kv : s->conns) { close(kv.second->fd); delete kv.second; }
    s->conns.clear();
  }
  s->cv.notify_all();
  close(s->lfd);
  close(s->ep);
  close(s->evfd);
  delete s;
}

// Waits up to timeout_ms for a parsed request. Returns 1 and fills conn / buf / len (free buf with vh_free),
// or 0 on timeout.
int vh_http_next(void* h, int timeout_ms, uint64_t* conn, char** buf, int* len) {
  auto* s = (Server*)h;
  std::unique_lock<std::mutex> lk(s->mu);
  if (s->reqs.empty()) s->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !s->reqs.empty() || s->stop.load(); });
  if (s->reqs.empty()) return 0;
  PendingReq r = std::move(s->reqs.front());
  s->reqs.pop_front();
  *conn = r.conn;
  *len = (int)r.blob.size();
  *buf = (char*)malloc(r.blob.size() + 1);
  memcpy(*buf, r.blob.data(), r.blob.size());
  (*buf)[r.blob.size()] = 0;
  return 1;
}

static const char* reason(int code) {
  switch (code) {
    case 200: return "OK"; case 204: return "No Content"; case 400: return "Bad Request"; case 401: return "Unauthorized";
    case 404: return "Not Found"; case 405: return "Method Not Allowed"; case 413: return "Payload Too Large";
    case 429: return "Too Many Requests"; case 500: return "Internal Server Error"; case 503: return "Service Unavailable";
  }
  return "Status";
}

// Complete response. extra_headers: zero or more "Name: value\r\n" lines (may be null).
int vh_http_respond(void* h, uint64_t conn, int status, const char* ctype, const char* body, int len, const char* extra_headers) {
  std::string head = "HTTP/1.1 " + std::to_string(status) + " " + reason(status) + "\r\nContent-Type: " + (ctype ? ctype : "application/json") +
                     "\r\nContent-Length: " + std::to_string(len) + "\r\nAccess-Control-Allow-Origin: *\r\n" + (extra_headers ? extra_headers : "") + "\r\n";
  head.append(body ? body : "", (size_t)len);
  return ((Server*)h)->enqueue(conn, head.data(), head.size(), true, false);
}

// Start of a streamed (chunked) response, e.g. text/event-stream.
int vh_http_stream_begin(void* h, uint64_t conn, int status, const char* ctype) {
  std::string head = "HTTP/1.1 " + std::to_string(status) + " " + reason(status) + "\r\nContent-Type: " + (ctype ? ctype : "text/event-stream") +
                     "\r\nCache-Control: no-cache\r\nTransfer-Encoding: chunked\r\nAccess-Control-Allow-Origin: *\r\nX-Accel-Buffering: no\r\n\r\n";
  auto* s = (Server*)h;
  {
    std::lock_guard<std::mutex> lk(s->mu);
    auto it = s->conns.find(conn);
    if (it != s->conns.end()) it->second->streaming = true;
  }
  return s->enqueue(conn, head.data(), head.size(), false, false);
}

int vh_http_stream_send(void* h, uint64_t conn, const char* data, int len) {
  if (len <= 0) return 0;
  char hdr[32];
  int n = snprintf(hdr, sizeof hdr, "%x\r\n", len);
  std::string chunk(hdr, (size_t)n);
  chunk.append(data, (size_t)len);
  chunk += "\r\n";
  return ((Server*)h)->enqueue(conn, chunk.data(), chunk.size(), false, false);
}

int vh_http_stream_end(void* h, uint64_t conn) {
  return ((Server*)h)->enqueue(conn, "0\r\n\r\n", 5, true, false);
}

// 1 while the client is still connected.
int vh_http_alive(void* h, uint64_t conn) {
  auto* s = (Server*)h;
  std::lock_guard<std::mutex> lk(s->mu);
  return s->conns.count(conn) ? 1 : 0;
}

void vh_http_stats(void* h, uint64_t* requests, uint64_t* dropped, int* connections) {
  auto* s = (Server*)h;
  std::lock_guard<std::mutex> lk(s->mu);
  *requests = s->n_requests.load();
  *dropped = s->n_dropped.load();
  *connections = (int)s->conns.size();
}

}  // extern "C"
