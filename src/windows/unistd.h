// Stand-in for <unistd.h> when the host runtime's portable parts (message model, codec,
// SArray, queues, Postoffice logic) are compiled with MSVC.  It maps the few POSIX names
// those files use onto the Windows C runtime; put this directory on the include path only on
// Windows.  The socket van itself (src/van/tcp_van.cc: epoll, Unix sockets) and the CUDA device
// plane are Linux-only, so a Windows build gets the loop van (single process) and the library
// types.  Same role as src/windows/unistd.h of the reference.
#ifndef PS_WINDOWS_UNISTD_H_
#define PS_WINDOWS_UNISTD_H_
#ifdef _WIN32

#include <direct.h>
#include <io.h>
#include <process.h>
#include <stdint.h>
#include <stdlib.h>
#include <windows.h>

// access() modes
#ifndef F_OK
#define F_OK 0
#define W_OK 2
#define R_OK 4
#define X_OK 0  // the CRT has no execute check: treat as existence
#endif

// standard descriptors
#ifndef STDIN_FILENO
#define STDIN_FILENO 0
#define STDOUT_FILENO 1
#define STDERR_FILENO 2
#endif

typedef intptr_t ssize_t;
typedef int pid_t;
typedef unsigned int useconds_t;

#define access _access
#define chdir _chdir
#define close _close
#define dup _dup
#define dup2 _dup2
#define getcwd _getcwd
#define getpid _getpid
#define isatty _isatty
#define lseek _lseek
#define read _read
#define rmdir _rmdir
#define unlink _unlink
#define write _write

static inline unsigned int sleep(unsigned int seconds) {
  Sleep(seconds * 1000u);
  return 0;
}
static inline int usleep(useconds_t usec) {
  // Sleep() has millisecond granularity: round up so that a short wait still yields
  Sleep((usec + 999u) / 1000u);
  return 0;
}
static inline int gethostname_utf8(char* name, size_t len) {
  DWORD n = (DWORD)len;
  return GetComputerNameA(name, &n) ? 0 : -1;
}

#endif  // _WIN32
#endif  // PS_WINDOWS_UNISTD_H_
