// Paged decode attention: the head sizes 80 to 128 (a translation unit of their own, compiled beside the
// one that holds the entry points and the smaller head sizes).
#include "attention_decode_kernel.cuh"

int cw_launch_decode_mid(int hd, const DecodeParams& p, int S, int splits, cudaStream_t stream) {
    switch (hd) {
        case 80: return launch_decode<80>(p, S, splits, stream);
        case 96: return launch_decode<96>(p, S, splits, stream);
        case 112: return launch_decode<112>(p, S, splits, stream);
        case 128: return launch_decode<128>(p, S, splits, stream);
    }
    return CW_ERR_UNSUPPORTED;
}

CW_TRACE_TU(attention_decode_mid)
