// Index arithmetic of the streaming layout, shared by host and device code.
//
// The streaming layout cuts a weight [n, k] into SLICES of 512 input channels and OCTS of
// 8 output rows.  One (slice, oct, plane) cell is 512 bytes = 32 lanes x 16 bytes: lane
// (r, j), r = lane >> 2 the row inside the oct, j = lane & 3 the 128-channel quarter of the
// slice, owns the 16 bytes of row 8*oct + r that cover channels 512*s + 128*j .. +127.
// Inside those 16 bytes the eight byte PAIRS are permuted by XOR with r: position i holds
// source byte 2*((i >> 1) ^ r) + (i & 1).  During a lookup of position i, lane (r, j) reads
// the table of channel-chunk c = 16*j + source byte, which lives in shared-memory bank
// 8*j + ((i >> 1) ^ r): the 32 lanes of a warp always touch 32 different banks.
//
// Cells are stored slice-major:  planes[s][oct][plane][lane][16].
// Scales and zeros follow the same ownership, two octs (a DUO, 16 rows) at a time so that a
// lane fetches both octs of a duo with one load:  meta[s][duo][pp][lane][oct & 1][u] (fp16),
// pp < q the plane's scale, pp == q the zero; u < gpw = 128 / g indexes the groups inside the
// lane's 128 channels BY BYTE POSITION, i.e. entry u belongs to source group
// u ^ (r >> log2(g/16)).  Rows >= n, channels >= k and their groups are stored as zeros.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define HLQ_HD __host__ __device__ __forceinline__
#else
#define HLQ_HD inline
#endif

namespace hlq {

constexpr int kSliceK = 512;       // input channels per slice
constexpr int kOctRows = 8;        // output rows per oct
constexpr int kCellBytes = 512;    // one plane of one oct of one slice
constexpr int kBlockRows = 32;     // rows per completion block (4 octs)

struct StreamDims {
    int n, k, g, q;
    int np;     // n rounded up to 32
    int kp;     // k rounded up to 512
    int slices; // kp / 512
    int octs;   // np / 8
    int duos;   // np / 16
    int blocks; // np / 32
    int gpw;    // groups per 128 channels: 128 / g
    int gshift; // log2(g / 16): 3, 2, 1 for g = 128, 64, 32
};

HLQ_HD bool stream_supported(int g) { return g == 128 || g == 64 || g == 32; }

HLQ_HD StreamDims stream_dims(int n, int k, int g, int q) {
    StreamDims d;
    d.n = n; d.k = k; d.g = g; d.q = q;
    d.np = (n + kBlockRows - 1) / kBlockRows * kBlockRows;
    d.kp = (k + kSliceK - 1) / kSliceK * kSliceK;
    d.slices = d.kp / kSliceK;
    d.octs = d.np / kOctRows;
    d.duos = d.octs / 2;
    d.blocks = d.np / kBlockRows;
    d.gpw = 128 / g;
    d.gshift = g == 128 ? 3 : (g == 64 ? 2 : 1);
    return d;
}

HLQ_HD int64_t stream_planes_bytes(const StreamDims &d) {
    return (int64_t)d.slices * d.octs * d.q * kCellBytes;
}
HLQ_HD int64_t stream_meta_elems(const StreamDims &d) {
    return (int64_t)d.slices * d.octs * (d.q + 1) * 32 * d.gpw;
}

// byte offset of position i of lane `lane` in cell (s, oct, p)
HLQ_HD int64_t stream_plane_offset(const StreamDims &d, int s, int oct, int p, int lane, int i) {
    return (((int64_t)s * d.octs + oct) * d.q + p) * kCellBytes + lane * 16 + i;
}
// source byte (0..15, within the lane's 16 source bytes) stored at position i for row r
HLQ_HD int stream_src_byte(int i, int r) { return 2 * ((i >> 1) ^ r) + (i & 1); }
// position that holds source byte b for row r (inverse of stream_src_byte)
HLQ_HD int stream_pos_of_src(int b, int r) { return 2 * ((b >> 1) ^ r) + (b & 1); }
// element offset of meta entry (s, oct, pp, lane, u)
HLQ_HD int64_t stream_meta_offset(const StreamDims &d, int s, int oct, int pp, int lane, int u) {
    const int64_t duo = oct >> 1;
    return (((((int64_t)s * d.duos + duo) * (d.q + 1) + pp) * 32 + lane) * 2 + (oct & 1)) * d.gpw + u;
}
// source group (within the lane's 128 channels) of positional sub-group u for row r
HLQ_HD int stream_src_group(const StreamDims &d, int u, int r) { return u ^ (r >> d.gshift); }

// Byte offset, inside one 256-byte table row, of the fp32 table of chunk c (8 channels)
// of a slice, c = 16*j + b:  bank 8*j + (b >> 1), bank-row b & 1.
HLQ_HD int table_chunk_offset(int c) {
    int j = c >> 4, b = c & 15;
    return 4 * (8 * j + (b >> 1)) + 128 * (b & 1);
}

}  // namespace hlq
