// Image decoding for the vision path without an image library: the scanline filters of PNG (the container and the inflate step
// stay in Python, models/vision.py) and a baseline JPEG decoder (Huffman-coded sequential DCT, 8-bit, 1 or 3 components, any
// sampling factors up to 2 x 2 per component, restart intervals).  The reference reads images through stb_image
// (common/stb_image.h behind server/server_llm.c:503); progressive and arithmetic-coded JPEG files are refused here with a message.
#include <cmath>
#include <cstring>
#include <vector>

#include "common.h"

namespace {

inline int paeth(int a, int b, int c) {
  const int p = a + b - c, pa = std::abs(p - a), pb = std::abs(p - b), pc = std::abs(p - c);
  return (pa <= pb && pa <= pc) ? a : (pb <= pc ? b : c);
}

struct Huff {                       // canonical code: for every length the first code and the index of its first symbol
  int maxcode[18], valptr[17], mincode[17];
  uint8_t vals[256];
  bool present = false;
};

struct Component { int id = 0, h = 1, v = 1, tq = 0, td = 0, ta = 0, pred = 0; std::vector<uint8_t> plane; int pw = 0, ph = 0; };

struct BitReader {
  const uint8_t* p; const uint8_t* end; uint32_t buf = 0; int cnt = 0; bool hit_marker = false;
  int bit() {
    if (cnt == 0) {
      int byte = 0;
      if (p < end && !hit_marker) {
        byte = *p++;
        if (byte == 0xFF) {
          const int nxt = p < end ? *p : 0xD9;
          if (nxt == 0x00) ++p;                                   // a stuffed zero after 0xFF
          else { hit_marker = true; --p; byte = 0; }             // a marker: feed zeros until the caller handles it
        }
      }
      buf = (uint32_t)byte; cnt = 8;
    }
    --cnt;
    return (buf >> cnt) & 1;
  }
  int bits(int n) { int v = 0; for (int i = 0; i < n; ++i) v = (v << 1) | bit(); return v; }
  void align() { cnt = 0; }
};

int decode_symbol(BitReader& br, const Huff& h) {
  int code = 0;
  for (int len = 1; len <= 16; ++len) {
    code = (code << 1) | br.bit();
    if (h.maxcode[len] >= 0 && code <= h.maxcode[len]) return h.vals[h.valptr[len] + code - h.mincode[len]];
  }
  return -1;
}

inline int extend(int v, int n) { return n == 0 ? 0 : (v < (1 << (n - 1)) ? v - (1 << n) + 1 : v); }

const uint8_t kZigzag[64] = {0, 1, 8, 16, 9, 2, 3, 10, 17, 24, 32, 25, 18, 11, 4, 5, 12, 19, 26, 33, 40, 48, 41, 34, 27, 20, 13, 6, 7, 14, 21, 28,
                             35, 42, 49, 56, 57, 50, 43, 36, 29, 22, 15, 23, 30, 37, 44, 51, 58, 59, 52, 45, 38, 31, 39, 46, 53, 60, 61, 54, 47, 55, 62, 63};

void idct8x8(const float* in, uint8_t* out, int stride) {
  static float c[8][8];
  static bool init = false;
  if (!init) {
    for (int x = 0; x < 8; ++x)
      for (int u = 0; u < 8; ++u) c[x][u] = (u == 0 ? std::sqrt(0.125f) : 0.5f) * std::cos((2 * x + 1) * u * 3.14159265358979323846f / 16.0f);
    init = true;
  }
  float tmp[64];
  for (int y = 0; y < 8; ++y)                                      // rows: tmp[y][x] = sum_u c[x][u] in[y][u]
    for (int x = 0; x < 8; ++x) { float s = 0.f; for (int u = 0; u < 8; ++u) s += c[x][u] * in[y * 8 + u]; tmp[y * 8 + x] = s; }
  for (int x = 0; x < 8; ++x)
    for (int y = 0; y < 8; ++y) {
      float s = 0.f;
      for (int v = 0; v < 8; ++v) s += c[y][v] * tmp[v * 8 + x];
      const int px = (int)std::lrintf(s + 128.0f);
      out[y * stride + x] = (uint8_t)(px < 0 ? 0 : (px > 255 ? 255 : px));
    }
}

inline int be16(const uint8_t* p) { return (p[0] << 8) | p[1]; }

}  // namespace

// Undo the scanline filters of a decompressed PNG stream in place: `rows` scanlines of 1 filter byte + `row_bytes` data bytes,
// `bpp` bytes per complete pixel (1 at least).  out: rows * row_bytes.  Returns 0, -1 on an unknown filter type.
GBH_API int gbh_png_unfilter(const uint8_t* raw, long rows, long row_bytes, int bpp, uint8_t* out) {
  for (long y = 0; y < rows; ++y) {
    const uint8_t* src = raw + y * (row_bytes + 1);
    const int ft = src[0];
    ++src;
    uint8_t* cur = out + y * row_bytes;
    const uint8_t* up = y > 0 ? cur - row_bytes : nullptr;
    for (long i = 0; i < row_bytes; ++i) {
      const int a = i >= bpp ? cur[i - bpp] : 0, b = up ? up[i] : 0, c = (up && i >= bpp) ? up[i - bpp] : 0;
      int v = src[i];
      switch (ft) {
        case 0: break;
        case 1: v += a; break;
        case 2: v += b; break;
        case 3: v += (a + b) >> 1; break;
        case 4: v += paeth(a, b, c); break;
        default: return gbh::fail("png: unknown filter type %d in row %ld", ft, y);
      }
      cur[i] = (uint8_t)v;
    }
  }
  return 0;
}

// Size of a JPEG image: 0 and *w, *h, *comps filled, or -1 with a message.
GBH_API int gbh_jpeg_info(const uint8_t* data, long n, int* w, int* h, int* comps) {
  if (n < 4 || data[0] != 0xFF || data[1] != 0xD8) return gbh::fail("jpeg: no SOI marker");
  long pos = 2;
  while (pos + 4 <= n) {
    if (data[pos] != 0xFF) { ++pos; continue; }
    const int m = data[pos + 1];
    if (m == 0xFF) { ++pos; continue; }
    pos += 2;
    if (m == 0xD8 || (m >= 0xD0 && m <= 0xD7) || m == 0x01) continue;
    const int len = be16(data + pos);
    if (len < 2 || pos + len > n) return gbh::fail("jpeg: truncated segment 0x%02X", m);
    if (m == 0xC0 || m == 0xC1) {
      if (len < 8) return gbh::fail("jpeg: short frame header");
      *h = be16(data + pos + 3); *w = be16(data + pos + 5); *comps = data[pos + 7];
      if ((long)*w * *h > (1L << 26)) return gbh::fail("jpeg: %d x %d is larger than this decoder accepts (64 Mpixel)", *w, *h);
      return 0;
    }
    if (m == 0xC2) return gbh::fail("jpeg: progressive files are not read (re-save as baseline)");
    if (m >= 0xC3 && m <= 0xCF && m != 0xC4 && m != 0xC8 && m != 0xCC) return gbh::fail("jpeg: coding process 0x%02X is not read (baseline only)", m);
    pos += len;
  }
  return gbh::fail("jpeg: no frame header");
}

// Decode a baseline JPEG into RGB bytes [h][w][3] (grey images are replicated).  0 on success.
GBH_API int gbh_jpeg_decode(const uint8_t* data, long n, uint8_t* rgb) {
  int W = 0, H = 0, nc = 0;
  if (gbh_jpeg_info(data, n, &W, &H, &nc) != 0) return -1;
  if (W <= 0 || H <= 0 || (nc != 1 && nc != 3)) return gbh::fail("jpeg: %d x %d with %d components is not read", W, H, nc);
  uint16_t qt[4][64] = {};
  Huff dc[4], ac[4];
  Component comp[3];
  int restart = 0, hmax = 1, vmax = 1;
  long pos = 2;
  bool decoded = false;
  while (pos + 4 <= n && !decoded) {
    if (data[pos] != 0xFF) { ++pos; continue; }
    const int m = data[pos + 1];
    if (m == 0xFF) { ++pos; continue; }
    pos += 2;
    if (m == 0xD8 || (m >= 0xD0 && m <= 0xD7) || m == 0x01) continue;
    if (m == 0xD9) break;
    const int len = be16(data + pos);
    if (len < 2 || pos + len > n) return gbh::fail("jpeg: truncated segment 0x%02X", m);
    const uint8_t* s = data + pos + 2;
    const uint8_t* send = data + pos + len;
    if (m == 0xDB) {
      while (s < send) {
        const int pq = s[0] >> 4, tq = s[0] & 15; ++s;
        if (tq > 3 || pq > 1 || s + (pq ? 128 : 64) > send) return gbh::fail("jpeg: bad quantisation table");
        for (int i = 0; i < 64; ++i) { qt[tq][kZigzag[i]] = pq ? (uint16_t)be16(s) : s[0]; s += pq ? 2 : 1; }
      }
    } else if (m == 0xC4) {
      while (s < send) {
        const int tc = s[0] >> 4, th = s[0] & 15; ++s;
        if (th > 3 || tc > 1 || s + 16 > send) return gbh::fail("jpeg: bad Huffman table id");
        Huff& h = tc ? ac[th] : dc[th];
        int counts[17] = {0}, total = 0;
        for (int i = 1; i <= 16; ++i) { counts[i] = s[i - 1]; total += counts[i]; }
        s += 16;
        if (total > 256 || s + total > send) return gbh::fail("jpeg: bad Huffman table");
        memcpy(h.vals, s, (size_t)total); s += total;
        int code = 0, k = 0;
        for (int l = 1; l <= 16; ++l) {
          h.valptr[l] = k; h.mincode[l] = code;
          code += counts[l]; k += counts[l];
          h.maxcode[l] = counts[l] ? code - 1 : -1;
          code <<= 1;
        }
        h.present = true;
      }
    } else if (m == 0xC0 || m == 0xC1) {
      if (len < 8 + 3 * nc) return gbh::fail("jpeg: short frame header");
      if (s[0] != 8) return gbh::fail("jpeg: %d-bit samples are not read", (int)s[0]);
      for (int i = 0; i < nc; ++i) {
        comp[i].id = s[6 + 3 * i]; comp[i].h = s[7 + 3 * i] >> 4; comp[i].v = s[7 + 3 * i] & 15; comp[i].tq = s[8 + 3 * i];
        if (comp[i].h < 1 || comp[i].h > 2 || comp[i].v < 1 || comp[i].v > 2 || comp[i].tq > 3) return gbh::fail("jpeg: sampling factors above 2 are not read");
        hmax = std::max(hmax, comp[i].h); vmax = std::max(vmax, comp[i].v);
      }
    } else if (m == 0xDD) {
      restart = be16(s);
    } else if (m == 0xDA) {
      if (len < 3) return gbh::fail("jpeg: short scan header");
      const int ns = s[0];
      if (len < 6 + 2 * ns) return gbh::fail("jpeg: short scan header");
      if (ns != nc) return gbh::fail("jpeg: a scan with %d of %d components is not read (non-interleaved files)", ns, nc);
      for (int i = 0; i < ns; ++i) {
        const int cid = s[1 + 2 * i];
        const int td = s[2 + 2 * i] >> 4, ta = s[2 + 2 * i] & 15;
        if (td > 3 || ta > 3) return gbh::fail("jpeg: bad Huffman table id in the scan header");
        for (int c = 0; c < nc; ++c) if (comp[c].id == cid) { comp[c].td = td; comp[c].ta = ta; }
      }
      const int mcu_w = 8 * hmax, mcu_h = 8 * vmax, mx = (W + mcu_w - 1) / mcu_w, my = (H + mcu_h - 1) / mcu_h;
      for (int c = 0; c < nc; ++c) {
        comp[c].pw = mx * comp[c].h * 8; comp[c].ph = my * comp[c].v * 8; comp[c].pred = 0;
        comp[c].plane.assign((size_t)comp[c].pw * comp[c].ph, 0);
        if (!dc[comp[c].td].present || !ac[comp[c].ta].present) return gbh::fail("jpeg: a scan names a Huffman table the file does not define");
      }
      BitReader br; br.p = data + pos + len; br.end = data + n;
      int until_restart = restart;
      for (int my_i = 0; my_i < my; ++my_i)
        for (int mx_i = 0; mx_i < mx; ++mx_i) {
          if (restart && until_restart == 0) {                    // RSTn: byte-align, skip the marker, reset the predictors
            br.align();
            const uint8_t* q = br.p;
            while (q + 1 < br.end && !(q[0] == 0xFF && q[1] >= 0xD0 && q[1] <= 0xD7)) ++q;
            if (q + 1 < br.end) br.p = q + 2;
            br.hit_marker = false;
            for (int c = 0; c < nc; ++c) comp[c].pred = 0;
            until_restart = restart;
          }
          for (int c = 0; c < nc; ++c)
            for (int by = 0; by < comp[c].v; ++by)
              for (int bx = 0; bx < comp[c].h; ++bx) {
                float blk[64] = {0};
                const int t = decode_symbol(br, dc[comp[c].td]);
                if (t < 0 || t > 11) return gbh::fail("jpeg: corrupt entropy-coded data");
                comp[c].pred += extend(br.bits(t), t);
                blk[0] = (float)(comp[c].pred * qt[comp[c].tq][0]);
                for (int k = 1; k < 64;) {
                  const int rs = decode_symbol(br, ac[comp[c].ta]);
                  if (rs < 0) return gbh::fail("jpeg: corrupt entropy-coded data");
                  const int r = rs >> 4, sz = rs & 15;
                  if (sz == 0) { if (r == 15) { k += 16; continue; } break; }
                  k += r;
                  if (k > 63) return gbh::fail("jpeg: corrupt entropy-coded data");
                  const int z = kZigzag[k];
                  blk[z] = (float)(extend(br.bits(sz), sz) * qt[comp[c].tq][z]);
                  ++k;
                }
                const int x0 = (mx_i * comp[c].h + bx) * 8, y0 = (my_i * comp[c].v + by) * 8;
                idct8x8(blk, comp[c].plane.data() + (size_t)y0 * comp[c].pw + x0, comp[c].pw);
              }
          if (restart) --until_restart;
        }
      decoded = true;
    }
    pos += len;
  }
  if (!decoded) return gbh::fail("jpeg: no scan found");
  for (int y = 0; y < H; ++y)
    for (int x = 0; x < W; ++x) {
      float v[3];
      for (int c = 0; c < nc; ++c) {
        // a subsampled plane is interpolated linearly between its sample centres (weights 3/4 and 1/4 at a factor of two, the
        // triangle filter most decoders use), clamped at the edge of the samples that cover the image
        const int vw = (W * comp[c].h + hmax - 1) / hmax, vh = (H * comp[c].v + vmax - 1) / vmax;
        float fx = (x + 0.5f) * comp[c].h / hmax - 0.5f, fy = (y + 0.5f) * comp[c].v / vmax - 0.5f;
        fx = fx < 0.f ? 0.f : (fx > vw - 1 ? (float)(vw - 1) : fx); fy = fy < 0.f ? 0.f : (fy > vh - 1 ? (float)(vh - 1) : fy);
        const int x0 = (int)fx, y0 = (int)fy, x1 = x0 + 1 < vw ? x0 + 1 : x0, y1 = y0 + 1 < vh ? y0 + 1 : y0;
        const float ax = fx - x0, ay = fy - y0;
        const uint8_t* pl = comp[c].plane.data();
        const size_t pw = (size_t)comp[c].pw;
        v[c] = (1 - ay) * ((1 - ax) * pl[y0 * pw + x0] + ax * pl[y0 * pw + x1]) + ay * ((1 - ax) * pl[y1 * pw + x0] + ax * pl[y1 * pw + x1]);
      }
      uint8_t* o = rgb + ((size_t)y * W + x) * 3;
      if (nc == 1) { o[0] = o[1] = o[2] = (uint8_t)std::lrintf(v[0]); continue; }
      const float Y = v[0], cb = v[1] - 128.0f, cr = v[2] - 128.0f;
      const float r = Y + 1.402f * cr, g = Y - 0.344136f * cb - 0.714136f * cr, b = Y + 1.772f * cb;
      const float ch[3] = {r, g, b};
      for (int i = 0; i < 3; ++i) { const int q = (int)std::lrintf(ch[i]); o[i] = (uint8_t)(q < 0 ? 0 : (q > 255 ? 255 : q)); }
    }
  return 0;
}
