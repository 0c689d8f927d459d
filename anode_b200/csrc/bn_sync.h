// Communicator handle of the synchronized batch-norm entry points.
#pragma once
#include <nccl.h>

struct AnodeSyncComm {
  ncclComm_t nccl;
  int rank, world;
  // optional in-kernel exchange: every rank's exchange buffer as mapped into this process
  unsigned long long *xchg[8];
  unsigned int xchg_channels;   // channels each buffer was sized for; 0 = not attached
  unsigned int epoch;           // calls made through the exchange so far (same on every rank)
};
