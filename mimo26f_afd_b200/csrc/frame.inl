// DS41RTE3 v3 frames on the host: what arrives at an expert rank and what it sends back.
// Layout and checks follow crates/mimo26-wire/src/layout.rs (field offsets 64-115, row contracts 4,360 / 8,192 bytes)
// and src/frame.rs (write_header 311-339, parse_header 341-393, RequestView::parse 868-955, return_header_seq 987-1030,
// seal / verify 405-455); the checksum is CRC32C (Castagnoli, reflected 0x82F63B78, src/crc32c.rs) over the whole
// frame with its own four bytes taken as zero. A request frame is
//     header 128 | row descriptors rows x 40 | route entries routes x 12 | hidden rows rows x stride (4096 E4M3 + 128 scales)
// and a return frame is header 128 | rows x 8192 bytes of BF16. Everything little-endian. This file is included into
// the library's single translation unit; nothing here touches the GPU.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstring>
#if defined(__x86_64__)
#include <nmmintrin.h>
#endif

namespace m26b_frame {

constexpr size_t kHeaderLen = 128, kDescLen = 40, kRouteLen = 12, kHiddenRow = 4096 + 128, kReturnRow = 8192;
constexpr uint16_t kVersion = 3, kKindRequest = 1, kKindReturn = 2;
constexpr uint16_t kDtypeBf16 = 1, kDtypeRowScaled = 5, kDtypeUe8m0K32 = 7;
constexpr uint32_t kFlagReturnRequired = (1u << 9) | (1u << 16);     // pre-summed on the rank, compact BF16
// header field offsets
constexpr size_t oMagic = 0, oVersion = 8, oKind = 10, oHeaderLen = 12, oRequestId = 16, oPlacement = 24, oLayer = 32,
                 oRowCount = 36, oDim = 40, oDtype = 44, oSourceKind = 46, oRouteCount = 48, oDescBytes = 52, oRouteBytes = 56,
                 oPayloadBytes = 60, oLogicalBytes = 68, oWireBytes = 76, oFlags = 84, oRowStride = 88, oStatus = 92,
                 oExecutor = 96, oTokenPos = 104, oSeq = 112, oCrc = 120;

inline void put16(uint8_t* b, size_t o, uint16_t v) { b[o] = uint8_t(v); b[o + 1] = uint8_t(v >> 8); }
inline void put32(uint8_t* b, size_t o, uint32_t v) { for (int i = 0; i < 4; ++i) b[o + i] = uint8_t(v >> (8 * i)); }
inline void put64(uint8_t* b, size_t o, uint64_t v) { for (int i = 0; i < 8; ++i) b[o + i] = uint8_t(v >> (8 * i)); }
inline uint16_t get16(const uint8_t* b, size_t o) { return uint16_t(b[o] | (b[o + 1] << 8)); }
inline uint32_t get32(const uint8_t* b, size_t o) { uint32_t v = 0; for (int i = 3; i >= 0; --i) v = (v << 8) | b[o + i]; return v; }
inline uint64_t get64(const uint8_t* b, size_t o) { uint64_t v = 0; for (int i = 7; i >= 0; --i) v = (v << 8) | b[o + i]; return v; }

struct CrcTable {
    uint32_t t[8][256];
    CrcTable() {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c & 1u) ? (c >> 1) ^ 0x82F63B78u : c >> 1;
            t[0][i] = c;
        }
        for (uint32_t i = 0; i < 256; ++i)
            for (int s = 1; s < 8; ++s) t[s][i] = (t[s - 1][i] >> 8) ^ t[0][t[s - 1][i] & 0xffu];
    }
};
#if defined(__x86_64__)
// The CPU's own CRC32C instruction where it exists (checked once at run time); the table path is its reference.
__attribute__((target("sse4.2"))) inline uint32_t crc_update_hw(uint32_t crc, const uint8_t* p, size_t n) {
    uint64_t c = crc;
    while (n && (reinterpret_cast<uintptr_t>(p) & 7u)) { c = _mm_crc32_u8(uint32_t(c), *p++); --n; }
    while (n >= 8) {
        uint64_t w;
        std::memcpy(&w, p, 8);
        c = _mm_crc32_u64(c, w);
        p += 8; n -= 8;
    }
    while (n--) c = _mm_crc32_u8(uint32_t(c), *p++);
    return uint32_t(c);
}
#endif
inline uint32_t crc_update_table(uint32_t crc, const uint8_t* p, size_t n);
inline uint32_t crc_update(uint32_t crc, const uint8_t* p, size_t n) {
#if defined(__x86_64__)
    static const bool hw = __builtin_cpu_supports("sse4.2");
    if (hw) return crc_update_hw(crc, p, n);
#endif
    return crc_update_table(crc, p, n);
}
inline uint32_t crc_update_table(uint32_t crc, const uint8_t* p, size_t n) {
    static const CrcTable T;
    while (n && (reinterpret_cast<uintptr_t>(p) & 7u)) { crc = (crc >> 8) ^ T.t[0][(crc ^ *p++) & 0xffu]; --n; }
    while (n >= 8) {                                        // slicing by eight
        uint64_t w;
        std::memcpy(&w, p, 8);
        w ^= crc;
        crc = T.t[7][w & 0xff] ^ T.t[6][(w >> 8) & 0xff] ^ T.t[5][(w >> 16) & 0xff] ^ T.t[4][(w >> 24) & 0xff] ^
              T.t[3][(w >> 32) & 0xff] ^ T.t[2][(w >> 40) & 0xff] ^ T.t[1][(w >> 48) & 0xff] ^ T.t[0][w >> 56];
        p += 8; n -= 8;
    }
    while (n--) crc = (crc >> 8) ^ T.t[0][(crc ^ *p++) & 0xffu];
    return crc;
}
inline uint32_t crc32c(const uint8_t* p, size_t n) { return ~crc_update(~0u, p, n); }
inline uint32_t crc32c_table(const uint8_t* p, size_t n) { return ~crc_update_table(~0u, p, n); }
// CRC32C of a frame with the header's checksum field taken as zero.
inline uint32_t frame_crc(const uint8_t* f, size_t n) {
    static const uint8_t zero[4] = {0, 0, 0, 0};
    uint32_t c = crc_update(~0u, f, oCrc);
    c = crc_update(c, zero, 4);
    c = crc_update(c, f + oCrc + 4, n - oCrc - 4);
    return ~c;
}

struct Header {
    uint16_t kind, dtype, source_kind;
    uint64_t request_id, placement_version, payload_bytes, logical_bytes, wire_bytes, executor_id, token_position, seq;
    uint32_t layer_id, row_count, dim, route_count, desc_bytes, route_bytes, flags, row_stride, status;
};

inline void write_header(uint8_t* b, const Header& h) {
    std::memset(b, 0, kHeaderLen);
    std::memcpy(b + oMagic, "DS41RTE3", 8);
    put16(b, oVersion, kVersion); put16(b, oKind, h.kind); put32(b, oHeaderLen, uint32_t(kHeaderLen));
    put64(b, oRequestId, h.request_id); put64(b, oPlacement, h.placement_version); put32(b, oLayer, h.layer_id);
    put32(b, oRowCount, h.row_count); put32(b, oDim, h.dim); put16(b, oDtype, h.dtype); put16(b, oSourceKind, h.source_kind);
    put32(b, oRouteCount, h.route_count); put32(b, oDescBytes, h.desc_bytes); put32(b, oRouteBytes, h.route_bytes);
    put64(b, oPayloadBytes, h.payload_bytes); put64(b, oLogicalBytes, h.logical_bytes); put64(b, oWireBytes, h.wire_bytes);
    put32(b, oFlags, h.flags); put32(b, oRowStride, h.row_stride); put32(b, oStatus, h.status);
    put64(b, oExecutor, h.executor_id); put64(b, oTokenPos, h.token_position); put64(b, oSeq, h.seq);
}

// The header checks of the reference, in its order. Returns nullptr or a message.
inline const char* parse_header(const uint8_t* f, size_t n, Header& h, char* msg, size_t msglen) {
    auto fail = [&](const char* fmt, unsigned long long a, unsigned long long b) { std::snprintf(msg, msglen, fmt, a, b); return msg; };
    if (n < kHeaderLen) return fail("frame too short: need %llu bytes, got %llu", kHeaderLen, n);
    if (std::memcmp(f + oMagic, "DS41RTE3", 8) != 0) return fail("bad frame magic%.0llu%.0llu", 0, 0);
    if (get16(f, oVersion) != kVersion) return fail("bad frame version %llu (want %llu)", get16(f, oVersion), kVersion);
    h.kind = get16(f, oKind);
    if (h.kind != kKindRequest && h.kind != kKindReturn) return fail("bad frame kind %llu%.0llu", h.kind, 0);
    if (get32(f, oHeaderLen) != kHeaderLen) return fail("bad header length %llu (want %llu)", get32(f, oHeaderLen), kHeaderLen);
    h.wire_bytes = get64(f, oWireBytes);
    if (n < h.wire_bytes) return fail("truncated frame: declared %llu bytes, got %llu", h.wire_bytes, n);
    if (n > h.wire_bytes) return fail("trailing bytes: declared %llu bytes, got %llu", h.wire_bytes, n);
    h.request_id = get64(f, oRequestId); h.placement_version = get64(f, oPlacement); h.layer_id = get32(f, oLayer);
    h.row_count = get32(f, oRowCount); h.dim = get32(f, oDim); h.dtype = get16(f, oDtype); h.source_kind = get16(f, oSourceKind);
    if (h.dtype < 1 || h.dtype > 7) return fail("bad code %llu in payload_dtype%.0llu", h.dtype, 0);
    if (h.source_kind < 1 || h.source_kind > 4) return fail("bad code %llu in source_kind%.0llu", h.source_kind, 0);
    h.route_count = get32(f, oRouteCount); h.desc_bytes = get32(f, oDescBytes); h.route_bytes = get32(f, oRouteBytes);
    h.payload_bytes = get64(f, oPayloadBytes); h.logical_bytes = get64(f, oLogicalBytes); h.flags = get32(f, oFlags);
    h.row_stride = get32(f, oRowStride); h.status = get32(f, oStatus);
    if (h.status > 1) return fail("bad code %llu in status%.0llu", h.status, 0);
    h.executor_id = get64(f, oExecutor); h.token_position = get64(f, oTokenPos); h.seq = get64(f, oSeq);
    return nullptr;
}

struct RequestView {
    Header h;
    const uint8_t* desc;      // rows x 40
    const uint8_t* routes;    // route_count x 12
    const uint8_t* hidden;    // rows x row_stride
};

// RequestView::parse: header, checksum, then the geometry and every descriptor / route entry.
inline const char* parse_request(const uint8_t* f, size_t n, bool check_crc, RequestView& v, char* msg, size_t msglen) {
    auto fail = [&](const char* fmt, unsigned long long a, unsigned long long b) { std::snprintf(msg, msglen, fmt, a, b); return msg; };
    if (const char* e = parse_header(f, n, v.h, msg, msglen)) return e;
    const Header& h = v.h;
    if (check_crc) {
        const uint32_t want = frame_crc(f, n), got = get32(f, oCrc);
        if (want != got) return fail("corrupt frame: CRC32C %08llx, header says %08llx", want, got);
    }
    if (h.kind != kKindRequest) return fail("bad frame kind %llu%.0llu", h.kind, 0);
    if (h.row_count == 0) return fail("row_count: want >= %llu, got %llu", 1, 0);
    const uint64_t rows = h.row_count, routes = h.route_count;
    if (h.desc_bytes != rows * kDescLen) return fail("row_descriptor_bytes: want %llu, got %llu", rows * kDescLen, h.desc_bytes);
    if (h.route_bytes != routes * kRouteLen) return fail("route_bytes: want %llu, got %llu", routes * kRouteLen, h.route_bytes);
    if (h.dim != 4096) return fail("hidden_dim: want %llu, got %llu", 4096, h.dim);
    if (h.dtype != kDtypeUe8m0K32 && h.dtype != kDtypeRowScaled) return fail("request_payload_dtype: want %llu, got %llu", kDtypeUe8m0K32, h.dtype);
    if (h.row_stride < 4096) return fail("row_stride_bytes: want >= %llu, got %llu", 4096, h.row_stride);
    if (h.payload_bytes != rows * h.row_stride) return fail("payload_bytes: want %llu, got %llu", rows * h.row_stride, h.payload_bytes);
    const uint64_t body = rows * kDescLen + routes * kRouteLen + rows * h.row_stride;
    if (n - kHeaderLen != body) return fail("body_len: want %llu, got %llu", body, n - kHeaderLen);
    v.desc = f + kHeaderLen;
    v.routes = v.desc + rows * kDescLen;
    v.hidden = v.routes + routes * kRouteLen;
    for (uint64_t i = 0; i < rows; ++i) {
        const uint8_t* d = v.desc + i * kDescLen;
        const uint16_t sk = get16(d, 8);
        if (sk < 1 || sk > 4) return fail("bad code %llu in source_kind (row %llu)", sk, i);
        if (uint64_t(get32(d, 28)) + get32(d, 32) > routes) return fail("row %llu: route range out of bounds%.0llu", i, 0);
    }
    for (uint64_t j = 0; j < routes; ++j)
        if (get32(v.routes + j * kRouteLen, 0) >= rows) return fail("route entry %llu names row %llu", j, get32(v.routes + j * kRouteLen, 0));
    return nullptr;
}

}  // namespace m26b_frame
