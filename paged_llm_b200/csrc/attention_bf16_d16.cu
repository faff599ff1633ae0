#define PL_DPAD 16
#include "attention_bf16.cuh"
