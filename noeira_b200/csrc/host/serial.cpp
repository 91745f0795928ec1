// Raw-mode serial port wrapper for the servo bus (termios / poll).  Counterpart of noeira/io/serial/native/nra_serial.c.
#include <cerrno>
#include <fcntl.h>
#include <poll.h>
#include <termios.h>
#include <unistd.h>

#include "host_api.h"

namespace {
speed_t baud_code(int baud) {
  switch (baud) {
    case 9600: return B9600;
    case 19200: return B19200;
    case 38400: return B38400;
    case 57600: return B57600;
    case 115200: return B115200;
    case 230400: return B230400;
    case 460800: return B460800;
    case 500000: return B500000;
    case 921600: return B921600;
    case 1000000: return B1000000;
    default: return 0;
  }
}
}  // namespace

extern "C" {

int nbh_serial_configure(int fd, int baud) {
  const speed_t sp = baud_code(baud);
  if (!sp) return -EINVAL;
  termios t;
  if (tcgetattr(fd, &t) != 0) return -errno;
  cfmakeraw(&t);
  t.c_cflag |= (CLOCAL | CREAD);
  t.c_cflag &= ~(PARENB | CSTOPB | CSIZE | CRTSCTS);
  t.c_cflag |= CS8;
  t.c_cc[VMIN] = 0;
  t.c_cc[VTIME] = 0;
  cfsetispeed(&t, sp);
  cfsetospeed(&t, sp);
  if (tcsetattr(fd, TCSANOW, &t) != 0) return -errno;
  return 0;
}

int nbh_serial_open(const char* path, int baud) {
  const int fd = open(path, O_RDWR | O_NOCTTY | O_NONBLOCK);
  if (fd < 0) return -errno;
  const int rc = nbh_serial_configure(fd, baud);
  if (rc != 0) { close(fd); return rc; }
  return fd;
}

int64_t nbh_serial_write(int fd, const void* data, size_t n) {
  size_t done = 0;
  while (done < n) {
    const ssize_t w = write(fd, (const char*)data + done, n - done);
    if (w < 0) {
      if (errno == EAGAIN || errno == EINTR) {
        pollfd p{fd, POLLOUT, 0};
        poll(&p, 1, 100);
        continue;
      }
      return -errno;
    }
    done += (size_t)w;
  }
  return (int64_t)done;
}

int64_t nbh_serial_read(int fd, void* out, size_t n, int timeout_ms) {
  size_t done = 0;
  while (done < n) {
    pollfd p{fd, POLLIN, 0};
    const int pr = poll(&p, 1, timeout_ms);
    if (pr == 0) break;                       // timeout: return what arrived
    if (pr < 0) { if (errno == EINTR) continue; return -errno; }
    const ssize_t r = read(fd, (char*)out + done, n - done);
    if (r < 0) { if (errno == EAGAIN || errno == EINTR) continue; return -errno; }
    if (r == 0) break;
    done += (size_t)r;
  }
  return (int64_t)done;
}

int nbh_serial_flush(int fd) { return tcflush(fd, TCIOFLUSH) == 0 ? 0 : -errno; }
int nbh_serial_close(int fd) { return close(fd) == 0 ? 0 : -errno; }

}  // extern "C"
