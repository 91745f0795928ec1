// Minimal HTTP/1.1 client over POSIX sockets with chunked-transfer decoding and gzip inflate (zlib); https:// through
// OpenSSL (server certificate and host name verified against the system trust store; NOEIRA_TLS_CA_FILE names an extra
// CA bundle, NOEIRA_TLS_INSECURE=1 switches verification off for tests against self-signed servers).
// Counterpart of noeira/io/native/nra_http.c (libcurl + zlib there; plain sockets + OpenSSL here).
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
#include <sys/time.h>
#include <openssl/err.h>
#include <openssl/ssl.h>
#include <openssl/x509v3.h>

#include "host_api.h"

namespace {

struct Url { std::string host, port, path; bool tls = false; };

int parse_url(const char* url, Url& u) {
  std::string s(url);
  if (s.rfind("https://", 0) == 0) { u.tls = true; s = s.substr(8); }
  else if (s.rfind("http://", 0) == 0) s = s.substr(7);
  else return -EINVAL;
  const size_t slash = s.find('/');
  std::string hp = slash == std::string::npos ? s : s.substr(0, slash);
  u.path = slash == std::string::npos ? "/" : s.substr(slash);
  const size_t colon = hp.rfind(':');
  if (colon != std::string::npos) { u.host = hp.substr(0, colon); u.port = hp.substr(colon + 1); }
  else { u.host = hp; u.port = u.tls ? "443" : "80"; }
  return u.host.empty() ? -EINVAL : 0;
}

// One connection: a socket, optionally wrapped in a TLS session.  Timeouts are socket timeouts (SO_RCVTIMEO /
// SO_SNDTIMEO), so the blocking OpenSSL calls return when the peer stalls.
struct Conn {
  int fd = -1;
  SSL_CTX* ctx = nullptr;
  SSL* ssl = nullptr;
  ~Conn() {
    if (ssl) { SSL_shutdown(ssl); SSL_free(ssl); }
    if (ctx) SSL_CTX_free(ctx);
    if (fd >= 0) close(fd);
  }
};

int tls_start(Conn& c, const std::string& host) {
  c.ctx = SSL_CTX_new(TLS_client_method());
  if (!c.ctx) return -ENOMEM;
  SSL_CTX_set_min_proto_version(c.ctx, TLS1_2_VERSION);
#ifdef SSL_OP_IGNORE_UNEXPECTED_EOF
  // "Connection: close" servers often drop the socket without a close_notify; the body length is checked by the HTTP layer
  SSL_CTX_set_options(c.ctx, SSL_OP_IGNORE_UNEXPECTED_EOF);
#endif
  const char* insecure = getenv("NOEIRA_TLS_INSECURE");
  const bool verify = !(insecure && insecure[0] == '1');
  if (verify) {
    SSL_CTX_set_default_verify_paths(c.ctx);
    if (const char* ca = getenv("NOEIRA_TLS_CA_FILE")) SSL_CTX_load_verify_locations(c.ctx, ca, nullptr);
    SSL_CTX_set_verify(c.ctx, SSL_VERIFY_PEER, nullptr);
  }
  c.ssl = SSL_new(c.ctx);
  if (!c.ssl) return -ENOMEM;
  SSL_set_tlsext_host_name(c.ssl, host.c_str());
  if (verify) {
    SSL_set_hostflags(c.ssl, X509_CHECK_FLAG_NO_PARTIAL_WILDCARDS);
    if (!SSL_set1_host(c.ssl, host.c_str())) return -EINVAL;
  }
  SSL_set_fd(c.ssl, c.fd);
  if (SSL_connect(c.ssl) != 1) return verify && SSL_get_verify_result(c.ssl) != X509_V_OK ? -EACCES : -ECONNABORTED;
  return 0;
}

int conn_send(Conn& c, const char* p, size_t n) {
  while (n) {
    ssize_t w;
    if (c.ssl) {
      w = SSL_write(c.ssl, p, (int)(n > (1u << 30) ? (1u << 30) : n));
      if (w <= 0) return -EIO;
    } else {
      w = send(c.fd, p, n, MSG_NOSIGNAL);
      if (w < 0) { if (errno == EINTR) continue; return errno == EAGAIN ? -ETIMEDOUT : -errno; }
    }
    p += w; n -= (size_t)w;
  }
  return 0;
}

// > 0 bytes read, 0 orderly end, < 0 error
ssize_t conn_recv(Conn& c, char* buf, size_t n) {
  if (c.ssl) {
    const int r = SSL_read(c.ssl, buf, (int)n);
    if (r > 0) return r;
    const int e = SSL_get_error(c.ssl, r);
    if (e == SSL_ERROR_ZERO_RETURN) return 0;
    if (e == SSL_ERROR_SYSCALL && errno == 0) return 0;     // peer closed without close_notify (Connection: close)
    return (e == SSL_ERROR_WANT_READ || errno == EAGAIN) ? -ETIMEDOUT : -EIO;
  }
  for (;;) {
    const ssize_t r = recv(c.fd, buf, n, 0);
    if (r < 0) { if (errno == EINTR) continue; return errno == EAGAIN ? -ETIMEDOUT : -errno; }
    return r;
  }
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
  Conn c;
  for (addrinfo* a = res; a; a = a->ai_next) {
    c.fd = socket(a->ai_family, a->ai_socktype, a->ai_protocol);
    if (c.fd < 0) continue;
    if (connect(c.fd, a->ai_addr, a->ai_addrlen) == 0) break;
    close(c.fd);
    c.fd = -1;
  }
  freeaddrinfo(res);
  if (c.fd < 0) return -ECONNREFUSED;
  timeval tv{timeout_ms / 1000, (timeout_ms % 1000) * 1000};
  setsockopt(c.fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  setsockopt(c.fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
  if (u.tls) {
    rc = tls_start(c, u.host);
    if (rc) return rc;
  }
  std::string req = std::string(method) + " " + u.path + " HTTP/1.1\r\nHost: " + u.host + "\r\nConnection: close\r\n" +
                    "Accept-Encoding: gzip\r\n";
  if (headers) req += headers;
  if (body_len) req += "Content-Length: " + std::to_string(body_len) + "\r\n";
  req += "\r\n";
  rc = conn_send(c, req.data(), req.size());
  if (!rc && body_len) rc = conn_send(c, (const char*)body, body_len);
  if (rc) return rc;
  std::string resp;
  char buf[16384];
  for (;;) {
    const ssize_t r = conn_recv(c, buf, sizeof(buf));
    if (r < 0) return (int)r;
    if (r == 0) break;
    resp.append(buf, (size_t)r);
  }
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
