/*
 * Layout of the control region at the start of every symmetric-heap arena (plain C, shared by
 * the kernels and by the host runtime's CPU stand-in of the device plane).
 */
#ifndef PS_DEVICE_CTRL_LAYOUT_H_
#define PS_DEVICE_CTRL_LAYOUT_H_
#include "ps/device/psdev.h"

/* flag_in[c][p] / flag_out[c][p] are written by rank p (remotely) and read by the owner of
 * the heap (locally). */
typedef struct psdev_ctrl {
  unsigned long long flag_in[PSDEV_NUM_CHANNELS][PSDEV_MAX_RANKS];
  unsigned long long flag_out[PSDEV_NUM_CHANNELS][PSDEV_MAX_RANKS];
  unsigned long long epoch[PSDEV_NUM_CHANNELS];
  unsigned int done[PSDEV_NUM_CHANNELS];
  int status[PSDEV_NUM_CHANNELS];
  /* who was late when a wait ran out: bit p set = rank p */
  unsigned int late_mask[PSDEV_NUM_CHANNELS];
} psdev_ctrl_t;

#endif /* PS_DEVICE_CTRL_LAYOUT_H_ */
