// Paged decode attention: the head sizes above 128 (a translation unit of their own, compiled beside
// the one that holds the entry points and the smaller head sizes).
#include "attention_decode_kernel.cuh"

int cw_launch_decode_large(int hd, const DecodeParams& p, int S, int splits, cudaStream_t stream) {
    switch (hd) {
        case 160: return launch_decode<160>(p, S, splits, stream);
        case 192: return launch_decode<192>(p, S, splits, stream);
        case 256: return launch_decode<256>(p, S, splits, stream);
    }
    return CW_ERR_UNSUPPORTED;
}

CW_TRACE_TU(attention_decode_large)
