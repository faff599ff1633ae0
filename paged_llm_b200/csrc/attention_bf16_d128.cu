#define PL_DPAD 128
#include "attention_bf16.cuh"
