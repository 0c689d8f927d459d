// Communicator handle of the synchronized batch-norm entry points.
#pragma once
#include <nccl.h>

struct AnodeSyncComm {
  ncclComm_t nccl;
  int rank, world;
};
