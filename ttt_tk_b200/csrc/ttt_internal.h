// Internal declarations shared by the translation units of libttt_mlp_b200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ttt_mlp_b200.h"

// Problem constants of the operator (kernels/ttt/ttt.cu:612-613 of the reference fixes the
// same ones): mini-batch of 64 tokens, head dimension 64, MLP hidden width 256.
constexpr int TTT_CS = 64;
constexpr int TTT_F = 64;
constexpr int TTT_HID = 256;
constexpr float TTT_LN_EPS = 1e-8f;

// Records `msg` as the calling thread's last error text and returns `code`.
int ttt_set_error(int code, const char* msg);

// Device-visible status word (pinned host memory, one per process).  Kernels write a
// non-zero code there when a bounded wait runs out; it stays set until taken.
int ttt_status_word(uint32_t** dev_ptr);

// Synchronise `stream`, then take (read and clear) the status word.
int ttt_check_status(cudaStream_t stream);

// Take the status word without synchronising (0 = nothing reported).
uint32_t ttt_take_status();

// Build a 2-D tensor map over a contiguous [rows][64] bf16 array with a 64 x 64 box and the
// 128-byte swizzle (the layout every 64 x 64 token tile of the operator has in memory).
int ttt_make_tile_map(CUtensorMap* map, const void* base, uint64_t rows);

// Limit of the device-side bounded waits in nanoseconds (TTT_B200_WAIT_LIMIT_MS, default 2000 ms).
uint64_t ttt_wait_limit_ns();

// Read and clear the device status word of ttt_b200_backward_noalloc (0 = nothing reported).
uint32_t ttt_noalloc_take_status();
