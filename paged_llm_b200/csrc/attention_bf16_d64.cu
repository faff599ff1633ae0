#define PL_DPAD 64
#include "attention_bf16.cuh"
