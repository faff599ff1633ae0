#define PL_DPAD 32
#include "attention_bf16.cuh"
