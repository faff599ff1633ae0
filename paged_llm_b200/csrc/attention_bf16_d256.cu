#define PL_DPAD 256
#include "attention_bf16.cuh"
