/*
 * Declarations of the part of the libzmq C API that the reference's ZMQ van uses
 * (src/zmq_van.h:37-248).  The development headers of libzmq are not installed on this
 * image; the shared library itself is (bundled with pyzmq), and the reference build for the
 * baseline arm links against it.  Signatures and constant values are those of libzmq 4.x.
 */
#ifndef BASELINE_SHIM_ZMQ_H_
#define BASELINE_SHIM_ZMQ_H_
#include <errno.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZMQ_HAUSNUMERO 156384712
#ifndef ETERM
#define ETERM (ZMQ_HAUSNUMERO + 53)
#endif

/* context options */
#define ZMQ_IO_THREADS 1
#define ZMQ_MAX_SOCKETS 2
/* socket types */
#define ZMQ_PAIR 0
#define ZMQ_DEALER 5
#define ZMQ_ROUTER 6
/* socket options */
#define ZMQ_IDENTITY 5
#define ZMQ_LINGER 17
#define ZMQ_SNDHWM 23
/* send/recv flags */
#define ZMQ_DONTWAIT 1
#define ZMQ_SNDMORE 2

typedef struct zmq_msg_t {
#if defined(__GNUC__) || defined(__clang__)
  unsigned char _[64] __attribute__((aligned(sizeof(void*))));
#else
  unsigned char _[64];
#endif
} zmq_msg_t;

typedef void(zmq_free_fn)(void* data, void* hint);

void* zmq_ctx_new(void);
int zmq_ctx_set(void* context, int option, int optval);
int zmq_ctx_destroy(void* context);
void* zmq_socket(void* context, int type);
int zmq_close(void* s);
int zmq_setsockopt(void* s, int option, const void* optval, size_t optvallen);
int zmq_bind(void* s, const char* addr);
int zmq_connect(void* s, const char* addr);
int zmq_msg_init(zmq_msg_t* msg);
int zmq_msg_init_data(zmq_msg_t* msg, void* data, size_t size, zmq_free_fn* ffn, void* hint);
int zmq_msg_send(zmq_msg_t* msg, void* s, int flags);
int zmq_msg_recv(zmq_msg_t* msg, void* s, int flags);
int zmq_msg_close(zmq_msg_t* msg);
void* zmq_msg_data(zmq_msg_t* msg);
size_t zmq_msg_size(const zmq_msg_t* msg);
int zmq_msg_more(const zmq_msg_t* msg);
const char* zmq_strerror(int errnum);
int zmq_errno(void);

#ifdef __cplusplus
}
#endif
#endif /* BASELINE_SHIM_ZMQ_H_ */
