// placeholder, replaced below
#pragma once
#include "comum.cuh"
namespace jt {
static int atencao_frente(int, const int8_t*, const int8_t*, int*, int16_t*, uint8_t*, int, int, int, int, int, int, cudaStream_t) { return (int)cudaErrorNotSupported; }
static int atencao_tras(int, const int8_t*, const int8_t*, const int8_t*, const int8_t*, const uint8_t*, int*, int16_t*, int, int, int, int, int, int, int, cudaStream_t) { return (int)cudaErrorNotSupported; }
}
