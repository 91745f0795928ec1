// Minimal HTTP/1.1 client over POSIX sockets with chunked-transfer decoding and gzip inflate (zlib).
// Counterpart of noeira/io/native/nra_http.c (libcurl + zlib there; plain sockets here, http:// only — there is no TLS
// library in this image, https URLs return -EPROTONOSUPPORT).
#include <arpa/inet.h>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <netdb.h>
#include <poll.h>
#include <string>
#include <sys/socket.h>
#include <unistd.h>
#include <zlib.h>

#include "host_api.h"

namespace {

struct Url { std::string host, port, path; };

int parse_url(const char* url, Url& u) {
  std::string s(url);
  if (s.rfind("https://", 0) == 0) return -EPROTONOSUPPORT;
  if (s.rfind("http://", 0) != 0) return -EINVAL;
  s = s.substr(7);
  const size_t slash = s.find('/');
  std::string hp = slash == std::string::npos ? s : s.substr(0, slash);
  u.path = slash == std::string::npos ? "/" : s.substr(slash);
  const size_t colon = hp.rfind(':');
  if (colon != std::string::npos) { u.host = hp.substr(0, colon); u.port = hp.substr(colon + 1); }
  else { u.host = hp; u.port = "80"; }
  return u.host.empty() ? -EINVAL : 0;
}

int wait_fd(int fd, short ev, int timeout_ms) {
  pollfd p{fd, ev, 0};
  const int r = poll(&p, 1, timeout_ms);
  if (r == 0) return -ETIMEDOUT;
  if (r < 0) return -errno;
  return 0;
}

int send_all(int fd, const char* p, size_t n, int timeout_ms) {
  while (n) {
    int rc = wait_fd(fd, POLLOUT, timeout_ms);
    if (rc) return rc;
    const ssize_t w = send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) { if (errno == EINTR || errno == EAGAIN) continue; return -errno; }
    p += w; n -= (size_t)w;
  }
  return 0;
}

std::string lower(std::string s) { for (auto& c : s) c = (char)tolower(c); return s; }

bool header_value(const std::string& head, const char* name, std::string& out) {
  const std::string h = lower(head), key = std::string("\r\n") + lower(name) + ":";
  const size_t p = h.find(key);
  if (p == std::string::npos) return false;
  size_t b = p + key.size();
  const size_t e = head.find("\r\n", b);
  out = head.substr(b, e - b);
  while (!out.empty() && out.front() == ' ') out.erase(out.begin());
  while (!out.empty() && (out.back() == ' ' || out.back() == '\r')) out.pop_back();
  return true;
}

int dechunk(const std::string& in, std::string& out) {
  size_t p = 0;
  for (;;) {
    const size_t e = in.find("\r\n", p);
    if (e == std::string::npos) return -EBADMSG;
    const unsigned long n = strtoul(in.substr(p, e - p).c_str(), nullptr, 16);
    p = e + 2;
    if (n == 0) return 0;
    if (p + n > in.size()) return -EBADMSG;
    out.append(in, p, n);
    p += n + 2;
  }
}

}  // namespace

extern "C" {

void nbh_free(void* p) { free(p); }

int64_t nbh_gzip_inflate(const void* src, size_t n, void** out, size_t* out_len) {
  z_stream zs;
  memset(&zs, 0, sizeof(zs));
  if (inflateInit2(&zs, 15 + 32) != Z_OK) return -ENOMEM;   // +32: zlib or gzip header, detected
  size_t cap = n * 4 + 1024, len = 0;
  uint8_t* buf = (uint8_t*)malloc(cap);
  if (!buf) { inflateEnd(&zs); return -ENOMEM; }
  zs.next_in = (Bytef*)src;
  zs.avail_in = (uInt)n;
  int rc;
  do {
    if (len == cap) {
      cap *= 2;
      uint8_t* nb = (uint8_t*)realloc(buf, cap);
      if (!nb) { free(buf); inflateEnd(&zs); return -ENOMEM; }
      buf = nb;
    }
    zs.next_out = buf + len;
    zs.avail_out = (uInt)(cap - len);
    rc = inflate(&zs, Z_NO_FLUSH);
    len = cap - zs.avail_out;
  } while (rc == Z_OK);
  inflateEnd(&zs);
  if (rc != Z_STREAM_END) { free(buf); return -EBADMSG; }
  *out = buf;
  *out_len = len;
  return (int64_t)len;
}

int nbh_http_request(const char* method, const char* url, const char* headers, const void* body, size_t body_len,
                     int timeout_ms, void** out_body, size_t* out_len) {
  Url u;
  int rc = parse_url(url, u);
  if (rc) return rc;
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(u.host.c_str(), u.port.c_str(), &hints, &res) != 0 || !res) return -EHOSTUNREACH;
  int fd = -1;
  for (addrinfo* a = res; a; a = a->ai_next) {
    fd = socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (fd < 0) continue;
    if (connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
    close(fd);
    fd = -1;
  }
  freeaddrinfo(res);
  if (fd < 0) return -ECONNREFUSED;
  std::string req = std::string(method) + " " + u.path + " HTTP/1.1\r\nHost: " + u.host + "\r\nConnection: close\r\n" +
                    "Accept-Encoding: gzip\r\n";
  if (headers) req += headers;
  if (body_len) req += "Content-Length: " + std::to_string(body_len) + "\r\n";
  req += "\r\n";
  rc = send_all(fd, req.data(), req.size(), timeout_ms);
  if (!rc && body_len) rc = send_all(fd, (const char*)body, body_len, timeout_ms);
  if (rc) { close(fd); return rc; }
  std::string resp;
  char buf[16384];
  for (;;) {
    rc = wait_fd(fd, POLLIN, timeout_ms);
    if (rc) { close(fd); return rc; }
    const ssize_t r = recv(fd, buf, sizeof(buf), 0);
    if (r < 0) { if (errno == EINTR || errno == EAGAIN) continue; close(fd); return -errno; }
    if (r == 0) break;
    resp.append(buf, (size_t)r);
  }
  close(fd);
  const size_t he = resp.find("\r\n\r\n");
  if (he == std::string::npos || resp.size() < 12) return -EBADMSG;
  const int status = atoi(resp.c_str() + 9);
  const std::string head = resp.substr(0, he + 2);
  std::string payload = resp.substr(he + 4), v;
  if (header_value(head, "transfer-encoding", v) && lower(v).find("chunked") != std::string::npos) {
    std::string d;
    rc = dechunk(payload, d);
    if (rc) return rc;
    payload.swap(d);
  }
  if (header_value(head, "content-encoding", v) && lower(v).find("gzip") != std::string::npos) {
    void* o = nullptr;
    size_t ol = 0;
    const int64_t g = nbh_gzip_inflate(payload.data(), payload.size(), &o, &ol);
    if (g < 0) return (int)g;
    *out_body = o;
    *out_len = ol;
    return status;
  }
  void* o = malloc(payload.size() ? payload.size() : 1);
  if (!o) return -ENOMEM;
  memcpy(o, payload.data(), payload.size());
  *out_body = o;
  *out_len = payload.size();
  return status;
}

}  // extern "C"
