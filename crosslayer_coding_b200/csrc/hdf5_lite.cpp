// Minimal HDF5 reader / writer for activation chunk files (no libhdf5, no h5py).
//
// Covers the subset the activation manifest format uses: groups `layer_N` holding 2-D datasets `inputs` and
// `targets` of float32 / float16 / uint16 (bf16 bit patterns), stored contiguous or row-chunked, optionally
// gzip-compressed (deflate, with or without the shuffle filter).
//
// Writer: superblock version 0, version-1 object headers, symbol-table groups (B-tree v1 + local heap),
// data layout version 3 - the layout libhdf5 / h5py produce with default settings, so the files open in h5py.
// Reader: superblock 0-3, object headers v1 and v2 (with continuation blocks), symbol-table groups and compact
// link-message groups, contiguous and chunked (B-tree v1) layouts, deflate + shuffle filters.  Dense groups
// (fractal heaps) and layout-v4 chunk indexes are reported as unsupported.
//
// Plain C ABI (ctypes-friendly).  Every function returns 0 / a handle on success; on failure it returns
// non-zero / null and clt_h5_last_error() describes the problem.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <zlib.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_error;
int fail(const std::string& msg) { g_error = msg; return -1; }

constexpr uint64_t UNDEF = 0xFFFFFFFFFFFFFFFFULL;
const unsigned char kSignature[8] = {0x89, 'H', 'D', 'F', '\r', '\n', 0x1a, '\n'};

enum DTypeCode { DT_F32 = 0, DT_F16 = 1, DT_U16 = 2, DT_I16 = 3, DT_F64 = 4, DT_U8 = 5, DT_I32 = 6, DT_OTHER = 99 };
int dtype_size(int code) {
  switch (code) {
    case DT_F32: case DT_I32: return 4;
    case DT_F16: case DT_U16: case DT_I16: return 2;
    case DT_F64: return 8;
    case DT_U8: return 1;
  }
  return 0;
}

// ============================================================================================ writer
struct Buf {
  std::vector<uint8_t> b;
  void u8(uint8_t v) { b.push_back(v); }
  void u16(uint16_t v) { for (int i = 0; i < 2; ++i) b.push_back(uint8_t(v >> (8 * i))); }
  void u32(uint32_t v) { for (int i = 0; i < 4; ++i) b.push_back(uint8_t(v >> (8 * i))); }
  void u64(uint64_t v) { for (int i = 0; i < 8; ++i) b.push_back(uint8_t(v >> (8 * i))); }
  void raw(const void* p, size_t n) { const uint8_t* q = static_cast<const uint8_t*>(p); b.insert(b.end(), q, q + n); }
  void pad8() { while (b.size() % 8) b.push_back(0); }
  size_t size() const { return b.size(); }
};

struct ChunkRec { uint64_t row0; uint64_t addr; uint32_t nbytes; };

struct DatasetRec {
  std::string name;
  uint64_t rows, cols;
  int dtype;
  uint64_t chunk_rows;  // 0 = contiguous
  int gzip;
  uint64_t data_addr = 0, data_size = 0;
  std::vector<ChunkRec> chunks;
  uint64_t header_addr = 0;
};

struct GroupRec {
  std::string name;
  std::vector<DatasetRec> datasets;
  uint64_t header_addr = 0;
};

struct Writer {
  FILE* fp = nullptr;
  std::string path, tmp_path;
  uint64_t pos = 0;
  std::vector<GroupRec> groups;

  bool put(const void* p, size_t n) {
    if (n && fwrite(p, 1, n, fp) != n) return false;
    pos += n;
    return true;
  }
  bool align8() {
    static const uint8_t z[8] = {0};
    const size_t padn = (8 - pos % 8) % 8;
    return put(z, padn);
  }
  uint64_t emit(const Buf& b) {
    align8();
    const uint64_t at = pos;
    put(b.b.data(), b.b.size());
    return at;
  }
};

void datatype_message(Buf& m, int dtype) {
  const int size = dtype_size(dtype);
  if (dtype == DT_F32 || dtype == DT_F16 || dtype == DT_F64) {
    m.u8(0x11);  // version 1, class 1 (floating point)
    m.u8(0x20);  // little endian, implied mantissa msb
    m.u8(uint8_t(size * 8 - 1));  // sign bit position
    m.u8(0);
    m.u32(size);
    m.u16(0);
    m.u16(uint16_t(size * 8));
    if (dtype == DT_F32) { m.u8(23); m.u8(8); m.u8(0); m.u8(23); m.u32(127); }
    else if (dtype == DT_F16) { m.u8(10); m.u8(5); m.u8(0); m.u8(10); m.u32(15); }
    else { m.u8(52); m.u8(11); m.u8(0); m.u8(52); m.u32(1023); }
  } else {
    m.u8(0x10);  // version 1, class 0 (fixed point)
    m.u8((dtype == DT_I16 || dtype == DT_I32) ? 0x08 : 0x00);  // little endian; bit 3 = signed
    m.u8(0); m.u8(0);
    m.u32(size);
    m.u16(0);
    m.u16(uint16_t(size * 8));
  }
}

void add_message(Buf& hdr, uint16_t type, const Buf& body, uint8_t flags = 0) {
  Buf b = body;
  b.pad8();
  hdr.u16(type);
  hdr.u16(uint16_t(b.size()));
  hdr.u8(flags);
  hdr.u8(0); hdr.u8(0); hdr.u8(0);
  hdr.raw(b.b.data(), b.size());
}

Buf object_header(const Buf& messages, int nmsg) {
  Buf h;
  h.u8(1); h.u8(0);
  h.u16(uint16_t(nmsg));
  h.u32(1);  // reference count
  h.u32(uint32_t(messages.size()));
  h.u32(0);  // pad the 12-byte prefix to 16 so messages are 8-aligned
  h.raw(messages.b.data(), messages.size());
  return h;
}

// B-tree v1 for chunked raw data: one leaf node when it fits, otherwise leaves under one level-1 node.
uint64_t write_chunk_btree(Writer& w, const DatasetRec& ds, int elem_size) {
  const size_t kMax = 64;  // 2 * default indexed-storage K (32)
  auto key = [&](Buf& b, uint32_t nbytes, uint64_t row0) {
    b.u32(nbytes); b.u32(0);
    b.u64(row0); b.u64(0); b.u64(0);  // offsets: row, col, element
  };
  auto node = [&](int level, const std::vector<ChunkRec>& recs, uint64_t end_row) {
    Buf b;
    b.raw("TREE", 4);
    b.u8(1); b.u8(uint8_t(level));
    b.u16(uint16_t(recs.size()));
    b.u64(UNDEF); b.u64(UNDEF);
    for (const ChunkRec& c : recs) { key(b, c.nbytes, c.row0); b.u64(c.addr); }
    key(b, 0, end_row);
    return w.emit(b);
  };
  const uint64_t end_row = ((ds.rows + ds.chunk_rows - 1) / ds.chunk_rows) * ds.chunk_rows;
  (void)elem_size;
  if (ds.chunks.size() <= kMax) return node(0, ds.chunks, end_row);
  std::vector<ChunkRec> upper;
  for (size_t i = 0; i < ds.chunks.size(); i += kMax) {
    std::vector<ChunkRec> part(ds.chunks.begin() + i, ds.chunks.begin() + std::min(ds.chunks.size(), i + kMax));
    const uint64_t part_end = (i + kMax < ds.chunks.size()) ? ds.chunks[i + kMax].row0 : end_row;
    ChunkRec r{part.front().row0, node(0, part, part_end), part.front().nbytes};
    upper.push_back(r);
  }
  return node(1, upper, end_row);
}

uint64_t write_dataset_header(Writer& w, DatasetRec& ds) {
  const int es = dtype_size(ds.dtype);
  Buf msgs;
  int n = 0;
  {  // dataspace v1
    Buf m; m.u8(1); m.u8(2); m.u8(0); m.u8(0); m.u32(0); m.u64(ds.rows); m.u64(ds.cols);
    add_message(msgs, 0x0001, m); ++n;
  }
  { Buf m; datatype_message(m, ds.dtype); add_message(msgs, 0x0003, m, 1); ++n; }
  {  // fill value v2: allocation early for chunked/late for contiguous is irrelevant here; undefined fill value
    Buf m; m.u8(2); m.u8(ds.chunk_rows ? 3 : 2); m.u8(0); m.u8(0);
    add_message(msgs, 0x0005, m); ++n;
  }
  if (ds.chunk_rows && ds.gzip > 0) {
    Buf m; m.u8(1); m.u8(1); m.u16(0); m.u32(0);
    m.u16(1);  // deflate
    m.u16(0);  // no name
    m.u16(1);  // optional filter
    m.u16(1);  // one client value
    m.u32(uint32_t(ds.gzip));
    m.u32(0);  // padding for an odd number of client values
    add_message(msgs, 0x000B, m); ++n;
  }
  {  // data layout v3
    Buf m; m.u8(3);
    if (ds.chunk_rows) {
      const uint64_t bt = write_chunk_btree(w, ds, es);
      m.u8(2); m.u8(3); m.u64(bt);
      m.u32(uint32_t(ds.chunk_rows)); m.u32(uint32_t(ds.cols)); m.u32(uint32_t(es));
    } else {
      m.u8(1); m.u64(ds.data_size ? ds.data_addr : UNDEF); m.u64(ds.data_size);
    }
    add_message(msgs, 0x0008, m); ++n;
  }
  ds.header_addr = w.emit(object_header(msgs, n));
  return ds.header_addr;
}

// Symbol-table group: local heap with the names, one SNOD leaf, one B-tree node, object header.
uint64_t write_group(Writer& w, std::vector<std::pair<std::string, uint64_t>> children) {
  std::sort(children.begin(), children.end());
  Buf heap_data;
  heap_data.u64(0);  // offset 0: empty name
  std::vector<uint64_t> name_off;
  for (auto& c : children) {
    name_off.push_back(heap_data.size());
    heap_data.raw(c.first.c_str(), c.first.size() + 1);
    heap_data.pad8();
  }
  // free block at the end (libhdf5 expects a well-formed free list or UNDEF)
  const uint64_t data_size = heap_data.size();
  const uint64_t heap_data_addr = w.emit(heap_data);
  Buf heap;
  heap.raw("HEAP", 4); heap.u8(0); heap.u8(0); heap.u8(0); heap.u8(0);
  heap.u64(data_size); heap.u64(UNDEF); heap.u64(heap_data_addr);
  const uint64_t heap_addr = w.emit(heap);
  Buf snod;
  snod.raw("SNOD", 4); snod.u8(1); snod.u8(0); snod.u16(uint16_t(children.size()));
  for (size_t i = 0; i < children.size(); ++i) {
    snod.u64(name_off[i]); snod.u64(children[i].second); snod.u32(0); snod.u32(0); snod.u64(0); snod.u64(0);
  }
  // a symbol node always reserves 2K entries (K = 64 in this writer's superblock)
  for (size_t i = children.size(); i < 128; ++i) { for (int k = 0; k < 5; ++k) snod.u64(0); }
  const uint64_t snod_addr = w.emit(snod);
  Buf tree;
  tree.raw("TREE", 4); tree.u8(0); tree.u8(0); tree.u16(children.empty() ? 0 : 1);
  tree.u64(UNDEF); tree.u64(UNDEF);
  tree.u64(0);  // key 0: empty string
  if (!children.empty()) { tree.u64(snod_addr); tree.u64(name_off.back()); }
  // reserve the full node: 2K children + 2K+1 keys with K = 16
  while (tree.size() < 24 + 8 * (2 * 16 + 2 * 16 + 1)) tree.u64(0);
  const uint64_t tree_addr = w.emit(tree);
  Buf msgs, m;
  m.u64(tree_addr); m.u64(heap_addr);
  add_message(msgs, 0x0011, m);
  return w.emit(object_header(msgs, 1));
}

bool deflate_chunk(const uint8_t* src, size_t n, int level, std::vector<uint8_t>& out) {
  uLongf cap = compressBound(n);
  out.resize(cap);
  if (compress2(out.data(), &cap, src, n, level) != Z_OK) return false;
  out.resize(cap);
  return true;
}

// ============================================================================================ reader
struct DatasetInfo {
  uint64_t rows = 0, cols = 1;
  int rank = 0;
  int elem_size = 0;
  int type_class = -1;   // 0 fixed point, 1 float
  bool is_signed = false;
  int layout = 0;        // 1 contiguous, 2 chunked, 0 compact (data inline)
  uint64_t data_addr = UNDEF, data_size = 0;
  uint64_t btree_addr = UNDEF;
  uint64_t chunk_rows = 0, chunk_cols = 0;
  bool deflate = false, shuffle = false;
  std::vector<uint8_t> compact;
  // chunk index: row0 -> (address, stored bytes, filter mask); only single-column-chunk layouts
  std::vector<ChunkRec> chunks;
  std::vector<uint32_t> chunk_mask;
  bool chunks_loaded = false;
};

struct Reader {
  int fd = -1;
  const uint8_t* base = nullptr;
  uint64_t size = 0;
  int so = 8, sl = 8;  // size of offsets / lengths
  uint64_t base_addr = 0;
  uint64_t root_header = UNDEF;
  std::map<std::string, DatasetInfo> ds_cache;
  // one decompressed chunk per dataset path
  std::map<std::string, std::pair<uint64_t, std::vector<uint8_t>>> chunk_cache;
  std::mutex mu;

  bool ok(uint64_t off, uint64_t n) const { return off != UNDEF && off <= size && n <= size - off; }
  uint64_t rd(uint64_t off, int n) const {
    uint64_t v = 0;
    for (int i = 0; i < n; ++i) v |= uint64_t(base[off + i]) << (8 * i);
    return v;
  }
  uint64_t rd_off(uint64_t off) const {
    uint64_t v = rd(off, so);
    if (so < 8 && v == ((1ULL << (8 * so)) - 1)) return UNDEF;
    return v == UNDEF ? UNDEF : v + base_addr;
  }
};

struct Message { uint16_t type; uint64_t off; uint32_t size; uint8_t flags; };

bool read_messages(const Reader& r, uint64_t addr, std::vector<Message>& out) {
  if (!r.ok(addr, 16)) return false;
  if (memcmp(r.base + addr, "OHDR", 4) == 0) {  // version 2
    const uint8_t flags = r.base[addr + 5];
    uint64_t p = addr + 6;
    if (flags & 0x20) p += 16;
    if (flags & 0x10) p += 4;
    const int szlen = 1 << (flags & 3);
    const uint64_t chunk0 = r.rd(p, szlen);
    p += szlen;
    std::vector<std::pair<uint64_t, uint64_t>> blocks{{p, chunk0}};
    const bool tracked = flags & 0x04;
    for (size_t bi = 0; bi < blocks.size(); ++bi) {
      uint64_t q = blocks[bi].first, end = q + blocks[bi].second;
      if (bi > 0) { q += 4; end -= 4; }  // "OCHK" signature ... checksum
      else end = q + blocks[bi].second;
      if (!r.ok(q, end - q)) return false;
      while (q + 4 <= end) {
        Message m;
        m.type = r.base[q];
        m.size = uint32_t(r.rd(q + 1, 2));
        m.flags = r.base[q + 3];
        q += 4 + (tracked ? 2 : 0);
        m.off = q;
        if (q + m.size > end + 4) break;
        if (m.type == 0x10) blocks.push_back({r.rd_off(q), r.rd(q + r.so, r.sl)});
        else if (m.type != 0) out.push_back(m);
        q += m.size;
      }
    }
    return true;
  }
  if (r.base[addr] != 1) return false;
  const int nmsg = int(r.rd(addr + 2, 2));
  const uint64_t hsize = r.rd(addr + 8, 4);
  std::vector<std::pair<uint64_t, uint64_t>> blocks{{addr + 16, hsize}};
  int seen = 0;
  for (size_t bi = 0; bi < blocks.size() && seen < nmsg; ++bi) {
    uint64_t q = blocks[bi].first;
    const uint64_t end = q + blocks[bi].second;
    if (!r.ok(q, blocks[bi].second)) return false;
    while (q + 8 <= end && seen < nmsg) {
      Message m;
      m.type = uint16_t(r.rd(q, 2));
      m.size = uint32_t(r.rd(q + 2, 2));
      m.flags = r.base[q + 4];
      m.off = q + 8;
      ++seen;
      if (m.type == 0x10) blocks.push_back({r.rd_off(m.off), r.rd(m.off + r.so, r.sl)});
      else out.push_back(m);
      q += 8 + m.size;
    }
  }
  return true;
}

// children of a group object header: name -> object header address
bool list_group(const Reader& r, uint64_t header, std::vector<std::pair<std::string, uint64_t>>& out) {
  std::vector<Message> msgs;
  if (!read_messages(r, header, msgs)) return false;
  for (const Message& m : msgs) {
    if (m.type == 0x11) {  // symbol table: B-tree + heap
      const uint64_t btree = r.rd_off(m.off), heap = r.rd_off(m.off + r.so);
      if (!r.ok(heap, 8 + 2 * r.sl + r.so) || memcmp(r.base + heap, "HEAP", 4) != 0) return false;
      const uint64_t heap_data = r.rd_off(heap + 8 + 2 * r.sl);
      std::vector<uint64_t> stack{btree};
      while (!stack.empty()) {
        const uint64_t node = stack.back();
        stack.pop_back();
        if (!r.ok(node, 8)) return false;
        if (memcmp(r.base + node, "TREE", 4) == 0) {
          const int n = int(r.rd(node + 6, 2));
          uint64_t p = node + 8 + 2 * r.so;
          for (int i = 0; i < n; ++i) {
            p += r.sl;  // key
            stack.push_back(r.rd_off(p));
            p += r.so;
          }
        } else if (memcmp(r.base + node, "SNOD", 4) == 0) {
          const int n = int(r.rd(node + 6, 2));
          uint64_t p = node + 8;
          for (int i = 0; i < n; ++i) {
            const uint64_t name_off = r.rd(p, r.so);
            const uint64_t obj = r.rd_off(p + r.so);
            const char* nm = reinterpret_cast<const char*>(r.base + heap_data + name_off);
            out.emplace_back(std::string(nm), obj);
            p += 2 * r.so + 8 + 16;
          }
        } else {
          return false;
        }
      }
    } else if (m.type == 0x06) {  // link message (compact new-style group)
      uint64_t p = m.off;
      const uint8_t ver = r.base[p], flags = r.base[p + 1];
      (void)ver;
      p += 2;
      uint8_t link_type = 0;
      if (flags & 0x08) link_type = r.base[p++];
      if (flags & 0x04) p += 8;
      if (flags & 0x10) p += 1;
      const int lensz = 1 << (flags & 3);
      const uint64_t len = r.rd(p, lensz);
      p += lensz;
      std::string name(reinterpret_cast<const char*>(r.base + p), len);
      p += len;
      if (link_type == 0) out.emplace_back(name, r.rd_off(p));
    } else if (m.type == 0x02) {  // link info: dense storage is not supported
      const uint8_t flags = r.base[m.off + 1];
      uint64_t p = m.off + 2 + ((flags & 1) ? 8 : 0);
      const uint64_t fheap = r.rd_off(p);
      if (fheap != UNDEF) { g_error = "dense (fractal-heap) groups are not supported"; return false; }
    }
  }
  return true;
}

bool resolve(const Reader& r, const std::string& path, uint64_t& header) {
  header = r.root_header;
  size_t i = 0;
  while (i < path.size()) {
    while (i < path.size() && path[i] == '/') ++i;
    size_t j = i;
    while (j < path.size() && path[j] != '/') ++j;
    if (j == i) break;
    const std::string part = path.substr(i, j - i);
    std::vector<std::pair<std::string, uint64_t>> kids;
    if (!list_group(r, header, kids)) return false;
    bool found = false;
    for (auto& k : kids) if (k.first == part) { header = k.second; found = true; break; }
    if (!found) { g_error = "no such object: " + path; return false; }
    i = j;
  }
  return true;
}

bool load_chunk_index(const Reader& r, DatasetInfo& d) {
  if (d.chunks_loaded) return true;
  std::vector<uint64_t> stack{d.btree_addr};
  const int ndims = d.rank + 1;
  while (!stack.empty()) {
    const uint64_t node = stack.back();
    stack.pop_back();
    if (node == UNDEF) continue;
    if (!r.ok(node, 8 + 2 * r.so) || memcmp(r.base + node, "TREE", 4) != 0 || r.base[node + 4] != 1) {
      g_error = "bad chunk B-tree node";
      return false;
    }
    const int level = r.base[node + 5];
    const int n = int(r.rd(node + 6, 2));
    uint64_t p = node + 8 + 2 * r.so;
    const uint64_t key_size = 8 + 8ULL * ndims;
    for (int i = 0; i < n; ++i) {
      const uint32_t nbytes = uint32_t(r.rd(p, 4)), mask = uint32_t(r.rd(p + 4, 4));
      const uint64_t row0 = r.rd(p + 8, 8);
      const uint64_t col0 = d.rank > 1 ? r.rd(p + 16, 8) : 0;
      p += key_size;
      const uint64_t child = r.rd_off(p);
      p += r.so;
      if (level > 0) stack.push_back(child);
      else {
        if (col0 != 0) { g_error = "chunks that split the column axis are not supported"; return false; }
        d.chunks.push_back({row0, child, nbytes});
        d.chunk_mask.push_back(mask);
      }
    }
  }
  std::vector<size_t> order(d.chunks.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = i;
  std::sort(order.begin(), order.end(), [&](size_t a, size_t b) { return d.chunks[a].row0 < d.chunks[b].row0; });
  std::vector<ChunkRec> c2; std::vector<uint32_t> m2;
  for (size_t i : order) { c2.push_back(d.chunks[i]); m2.push_back(d.chunk_mask[i]); }
  d.chunks.swap(c2); d.chunk_mask.swap(m2);
  d.chunks_loaded = true;
  return true;
}

bool dataset_info(Reader& r, const std::string& path, DatasetInfo*& out) {
  auto it = r.ds_cache.find(path);
  if (it != r.ds_cache.end()) { out = &it->second; return true; }
  uint64_t header;
  if (!resolve(r, path, header)) return false;
  std::vector<Message> msgs;
  if (!read_messages(r, header, msgs)) { g_error = "cannot parse object header of " + path; return false; }
  DatasetInfo d;
  bool have_space = false, have_type = false, have_layout = false;
  for (const Message& m : msgs) {
    const uint64_t p = m.off;
    if (m.type == 0x01) {
      const uint8_t ver = r.base[p];
      d.rank = r.base[p + 1];
      const uint64_t dims = p + (ver == 1 ? 8 : 4);
      if (d.rank < 1 || d.rank > 2) { g_error = "only 1-D and 2-D datasets are supported"; return false; }
      d.rows = r.rd(dims, r.sl);
      d.cols = d.rank == 2 ? r.rd(dims + r.sl, r.sl) : 1;
      have_space = true;
    } else if (m.type == 0x03) {
      d.type_class = r.base[p] & 0x0F;
      d.is_signed = (r.base[p + 1] & 0x08) != 0;
      d.elem_size = int(r.rd(p + 4, 4));
      if (r.base[p + 1] & 0x01) { g_error = "big-endian data is not supported"; return false; }
      have_type = true;
    } else if (m.type == 0x08) {
      const uint8_t ver = r.base[p];
      if (ver == 3) {
        d.layout = r.base[p + 1];
        if (d.layout == 1) { d.data_addr = r.rd_off(p + 2); d.data_size = r.rd(p + 2 + r.so, r.sl); }
        else if (d.layout == 2) {
          const int nd = r.base[p + 2];
          d.btree_addr = r.rd_off(p + 3);
          const uint64_t dims = p + 3 + r.so;
          d.chunk_rows = r.rd(dims, 4);
          d.chunk_cols = nd >= 3 ? r.rd(dims + 4, 4) : 1;
        } else if (d.layout == 0) {
          const uint64_t n = r.rd(p + 2, 2);
          d.compact.assign(r.base + p + 4, r.base + p + 4 + n);
        }
      } else if (ver == 1 || ver == 2) {
        const int nd = r.base[p + 1];
        d.layout = r.base[p + 2];
        uint64_t q = p + 8;
        if (d.layout != 0) { (d.layout == 1 ? d.data_addr : d.btree_addr) = r.rd_off(q); q += r.so; }
        if (d.layout == 2) { d.chunk_rows = r.rd(q, 4); d.chunk_cols = nd >= 3 ? r.rd(q + 4, 4) : 1; }
        else if (d.layout == 1) { d.data_size = 0; }
      } else {
        g_error = "data layout message version " + std::to_string(ver) + " is not supported";
        return false;
      }
      have_layout = true;
    } else if (m.type == 0x0B) {
      const uint8_t ver = r.base[p];
      const int nf = r.base[p + 1];
      uint64_t q = p + (ver == 1 ? 8 : 2);
      for (int i = 0; i < nf; ++i) {
        const uint16_t id = uint16_t(r.rd(q, 2));
        uint16_t namelen = 0;
        if (ver == 1 || id >= 256) { namelen = uint16_t(r.rd(q + 2, 2)); q += 4; } else q += 2;
        q += 2;  // flags
        const uint16_t ncd = uint16_t(r.rd(q, 2));
        q += 2;
        q += ver == 1 ? ((namelen + 7) / 8) * 8 : namelen;
        q += 4ULL * ncd;
        if (ver == 1 && (ncd & 1)) q += 4;
        if (id == 1) d.deflate = true;
        else if (id == 2) d.shuffle = true;
        else { g_error = "unsupported filter id " + std::to_string(id); return false; }
      }
    }
  }
  if (!have_space || !have_type || !have_layout) { g_error = path + " is not a dataset"; return false; }
  if (d.layout == 1 && d.data_size == 0) d.data_size = d.rows * d.cols * d.elem_size;
  if (d.layout == 2) {
    if (d.chunk_cols != d.cols && d.rank == 2) { g_error = "chunks must span whole rows"; return false; }
    if (!load_chunk_index(r, d)) return false;
  }
  out = &(r.ds_cache[path] = std::move(d));
  return true;
}

// decompressed bytes of chunk `ci` (cached per dataset)
const uint8_t* chunk_data(Reader& r, const std::string& path, DatasetInfo& d, size_t ci) {
  const ChunkRec& c = d.chunks[ci];
  const uint64_t full = d.chunk_rows * d.cols * d.elem_size;
  const bool filtered = (d.deflate && !(d.chunk_mask[ci] & 1)) || d.shuffle;
  if (!r.ok(c.addr, c.nbytes)) { g_error = "chunk outside the file"; return nullptr; }
  if (!filtered) return r.base + c.addr;
  auto& slot = r.chunk_cache[path];
  if (slot.second.size() == full && slot.first == ci) return slot.second.data();
  std::vector<uint8_t> tmp(full);
  const uint8_t* src = r.base + c.addr;
  if (d.deflate && !(d.chunk_mask[ci] & 1)) {
    uLongf n = full;
    if (uncompress(tmp.data(), &n, src, c.nbytes) != Z_OK || n != full) { g_error = "inflate failed"; return nullptr; }
  } else {
    memcpy(tmp.data(), src, std::min<uint64_t>(full, c.nbytes));
  }
  const bool shuffled = d.shuffle && !(d.chunk_mask[ci] & (d.deflate ? 2 : 1));
  if (shuffled && d.elem_size > 1) {
    std::vector<uint8_t> un(full);
    const uint64_t n = full / d.elem_size;
    for (int b = 0; b < d.elem_size; ++b)
      for (uint64_t i = 0; i < n; ++i) un[i * d.elem_size + b] = tmp[b * n + i];
    tmp.swap(un);
  }
  slot.first = ci;
  slot.second.swap(tmp);
  return slot.second.data();
}

int read_rows_impl(Reader& r, const std::string& path, const uint64_t* rows, uint64_t n, bool all, uint8_t* out) {
  DatasetInfo* dp;
  if (!dataset_info(r, path, dp)) return -1;
  DatasetInfo& d = *dp;
  const uint64_t rb = d.cols * d.elem_size;
  if (all) n = d.rows;
  if (d.layout == 1 || d.layout == 0) {
    const uint8_t* src = d.layout == 1 ? (d.data_addr == UNDEF ? nullptr : r.base + d.data_addr) : d.compact.data();
    if (d.layout == 1 && d.data_addr != UNDEF && !r.ok(d.data_addr, d.rows * rb)) return fail("dataset outside the file");
    for (uint64_t i = 0; i < n; ++i) {
      const uint64_t row = all ? i : rows[i];
      if (row >= d.rows) return fail("row index out of range");
      if (src) memcpy(out + i * rb, src + row * rb, rb); else memset(out + i * rb, 0, rb);
    }
    return 0;
  }
  for (uint64_t i = 0; i < n; ++i) {
    const uint64_t row = all ? i : rows[i];
    if (row >= d.rows) return fail("row index out of range");
    const uint64_t want = (row / d.chunk_rows) * d.chunk_rows;
    size_t lo = 0, hi = d.chunks.size();
    while (lo < hi) { const size_t mid = (lo + hi) / 2; if (d.chunks[mid].row0 < want) lo = mid + 1; else hi = mid; }
    if (lo == d.chunks.size() || d.chunks[lo].row0 != want) { memset(out + i * rb, 0, rb); continue; }  // unallocated chunk
    const uint8_t* cd = chunk_data(r, path, d, lo);
    if (!cd) return -1;
    memcpy(out + i * rb, cd + (row - want) * rb, rb);
  }
  return 0;
}

}  // namespace

extern "C" {

const char* clt_h5_last_error() { return g_error.c_str(); }

// ---------------------------------------------------------------------------------------- writer API
void* clt_h5w_open(const char* path) {
  auto w = std::make_unique<Writer>();
  w->path = path;
  w->tmp_path = std::string(path) + ".tmp";
  w->fp = fopen(w->tmp_path.c_str(), "wb");
  if (!w->fp) { fail(std::string("cannot create ") + w->tmp_path); return nullptr; }
  uint8_t zeros[96] = {0};
  w->put(zeros, 96);  // superblock, written on close
  return w.release();
}

// data: rows x cols elements of `dtype`, C order.  chunk_rows == 0 stores the dataset contiguously;
// gzip_level > 0 compresses each chunk with deflate.
int clt_h5w_add_dataset(void* handle, const char* group, const char* name, const void* data, uint64_t rows, uint64_t cols,
                        int dtype, uint64_t chunk_rows, int gzip_level) {
  Writer& w = *static_cast<Writer*>(handle);
  const int es = dtype_size(dtype);
  if (es == 0) return fail("unsupported dtype code");
  if (gzip_level > 0 && chunk_rows == 0) chunk_rows = std::min<uint64_t>(std::max<uint64_t>(rows, 1), 16384);
  GroupRec* g = nullptr;
  for (auto& gr : w.groups) if (gr.name == group) g = &gr;
  if (!g) { w.groups.push_back(GroupRec{group, {}, 0}); g = &w.groups.back(); }
  DatasetRec ds;
  ds.name = name; ds.rows = rows; ds.cols = cols; ds.dtype = dtype; ds.chunk_rows = chunk_rows; ds.gzip = gzip_level;
  const uint8_t* src = static_cast<const uint8_t*>(data);
  const uint64_t rb = cols * es;
  if (chunk_rows == 0) {
    w.align8();
    ds.data_addr = w.pos;
    ds.data_size = rows * rb;
    if (!w.put(src, ds.data_size)) return fail("write failed");
  } else {
    std::vector<uint8_t> padded, packed;
    for (uint64_t r0 = 0; r0 < rows; r0 += chunk_rows) {
      const uint64_t nr = std::min(chunk_rows, rows - r0);
      const uint8_t* cptr = src + r0 * rb;
      if (nr < chunk_rows) {  // edge chunks are stored at full size
        padded.assign(chunk_rows * rb, 0);
        memcpy(padded.data(), cptr, nr * rb);
        cptr = padded.data();
      }
      const uint8_t* outp = cptr;
      uint64_t outn = chunk_rows * rb;
      if (gzip_level > 0) {
        if (!deflate_chunk(cptr, chunk_rows * rb, gzip_level, packed)) return fail("deflate failed");
        outp = packed.data();
        outn = packed.size();
      }
      w.align8();
      ds.chunks.push_back({r0, w.pos, uint32_t(outn)});
      if (!w.put(outp, outn)) return fail("write failed");
    }
  }
  g->datasets.push_back(std::move(ds));
  return 0;
}

int clt_h5w_close(void* handle) {
  std::unique_ptr<Writer> w(static_cast<Writer*>(handle));
  std::vector<std::pair<std::string, uint64_t>> root_children;
  for (auto& g : w->groups) {
    std::vector<std::pair<std::string, uint64_t>> kids;
    for (auto& ds : g.datasets) kids.emplace_back(ds.name, write_dataset_header(*w, ds));
    if (g.name.empty()) { for (auto& k : kids) root_children.push_back(k); continue; }
    root_children.emplace_back(g.name, write_group(*w, kids));
  }
  const uint64_t root = write_group(*w, root_children);
  w->align8();
  const uint64_t eof = w->pos;
  Buf sb;
  sb.raw(kSignature, 8);
  sb.u8(0); sb.u8(0); sb.u8(0); sb.u8(0); sb.u8(0);
  sb.u8(8); sb.u8(8); sb.u8(0);
  sb.u16(64);  // group leaf node K: a symbol node holds up to 128 entries
  sb.u16(16);  // group internal node K
  sb.u32(0);
  sb.u64(0); sb.u64(UNDEF); sb.u64(eof); sb.u64(UNDEF);
  sb.u64(0); sb.u64(root); sb.u32(0); sb.u32(0); sb.u64(0); sb.u64(0);  // root symbol table entry (not cached)
  int rc = 0;
  if (fseek(w->fp, 0, SEEK_SET) != 0 || fwrite(sb.b.data(), 1, sb.size(), w->fp) != sb.size()) rc = fail("cannot write superblock");
  if (fclose(w->fp) != 0 && rc == 0) rc = fail("close failed");
  if (rc == 0 && rename(w->tmp_path.c_str(), w->path.c_str()) != 0) rc = fail("rename failed");
  return rc;
}

// ---------------------------------------------------------------------------------------- reader API
void* clt_h5r_open(const char* path) {
  auto r = std::make_unique<Reader>();
  r->fd = open(path, O_RDONLY);
  if (r->fd < 0) { fail(std::string("cannot open ") + path); return nullptr; }
  struct stat st;
  if (fstat(r->fd, &st) != 0 || st.st_size < 96) { close(r->fd); fail("file too small to be HDF5"); return nullptr; }
  r->size = uint64_t(st.st_size);
  // MAP_POPULATE: the page tables are filled in one go at open time (read-ahead from disk when the file is not cached);
  // a batch assembly that touches tens of thousands of pages would otherwise take one minor fault per page
  void* mp = mmap(nullptr, r->size, PROT_READ, MAP_PRIVATE | MAP_POPULATE, r->fd, 0);
  if (mp == MAP_FAILED) mp = mmap(nullptr, r->size, PROT_READ, MAP_PRIVATE, r->fd, 0);
  if (mp == MAP_FAILED) { close(r->fd); fail("mmap failed"); return nullptr; }
  r->base = static_cast<const uint8_t*>(mp);
  uint64_t sb = 0;
  bool found = false;
  for (; sb + 96 <= r->size; sb = sb ? sb * 2 : 512) {
    if (memcmp(r->base + sb, kSignature, 8) == 0) { found = true; break; }
    if (sb > (1ULL << 24)) break;
  }
  auto bail = [&](const char* msg) -> void* { munmap(mp, r->size); close(r->fd); fail(msg); return nullptr; };
  if (!found) return bail("not an HDF5 file (signature missing)");
  const uint8_t ver = r->base[sb + 8];
  if (ver <= 1) {
    r->so = r->base[sb + 13];
    r->sl = r->base[sb + 14];
    uint64_t p = sb + 24 + (ver == 1 ? 4 : 0);
    r->base_addr = r->rd(p, r->so);
    p += 4 * r->so;
    r->root_header = r->rd_off(p + r->so);
  } else if (ver == 2 || ver == 3) {
    r->so = r->base[sb + 9];
    r->sl = r->base[sb + 10];
    uint64_t p = sb + 12;
    r->base_addr = r->rd(p, r->so);
    r->root_header = r->rd_off(p + 3 * r->so);
  } else {
    return bail("unsupported superblock version");
  }
  if (r->so != 8 || r->sl != 8) return bail("only 8-byte offsets/lengths are supported");
  return r.release();
}

void clt_h5r_close(void* handle) {
  std::unique_ptr<Reader> r(static_cast<Reader*>(handle));
  if (r->base) munmap(const_cast<uint8_t*>(r->base), r->size);
  if (r->fd >= 0) close(r->fd);
}

// Newline-separated child names of the group at `path` ("" or "/" for the root).  Returns the number of
// bytes needed (including the terminator); the list is written only when it fits.
long long clt_h5r_list(void* handle, const char* path, char* buf, long long buflen) {
  Reader& r = *static_cast<Reader*>(handle);
  std::lock_guard<std::mutex> lock(r.mu);
  uint64_t header;
  if (!resolve(r, path, header)) return -1;
  std::vector<std::pair<std::string, uint64_t>> kids;
  if (!list_group(r, header, kids)) { if (g_error.empty()) fail("cannot list group"); return -1; }
  std::string s;
  for (auto& k : kids) { s += k.first; s += '\n'; }
  if ((long long)s.size() + 1 <= buflen) memcpy(buf, s.c_str(), s.size() + 1);
  return (long long)s.size() + 1;
}

// info: rows, cols, elem_size, type_class (0 int, 1 float), is_signed, layout, chunk_rows, compressed
int clt_h5r_dataset_info(void* handle, const char* path, uint64_t* info) {
  Reader& r = *static_cast<Reader*>(handle);
  std::lock_guard<std::mutex> lock(r.mu);
  DatasetInfo* d;
  if (!dataset_info(r, path, d)) return -1;
  info[0] = d->rows; info[1] = d->cols; info[2] = uint64_t(d->elem_size); info[3] = uint64_t(d->type_class);
  info[4] = d->is_signed; info[5] = uint64_t(d->layout); info[6] = d->chunk_rows; info[7] = d->deflate ? 1 : 0;
  return 0;
}

int clt_h5r_read_rows(void* handle, const char* path, const uint64_t* rows, uint64_t n, void* out) {
  Reader& r = *static_cast<Reader*>(handle);
  std::lock_guard<std::mutex> lock(r.mu);
  return read_rows_impl(r, path, rows, n, false, static_cast<uint8_t*>(out));
}

// Gather `n` rows of each of `npaths` datasets (paths separated by '\n') into caller memory: row rows[i] of
// dataset p goes to dst_bases[p] + dst_pos[i] * dst_row_stride.  Contiguous datasets are copied straight from
// the mapped file by `nthreads` threads (the batch assembly of a training step is a few hundred thousand small
// row copies); filtered / chunked datasets take the serial path through the chunk cache.
int clt_h5r_scatter_rows(void* handle, const char* paths, int npaths, const uint64_t* rows, const int64_t* dst_pos, uint64_t n,
                         void* const* dst_bases, uint64_t dst_row_stride, int nthreads) {
  Reader& r = *static_cast<Reader*>(handle);
  std::lock_guard<std::mutex> lock(r.mu);
  // a job copies rows of one dataset: contiguous layout (src) or unfiltered chunks (file address per chunk of chunk_rows rows)
  struct Job { const uint8_t* src; uint8_t* dst; uint64_t rb; uint64_t chunk_rows; std::vector<uint64_t> chunk_addr; };
  std::vector<Job> jobs;
  std::vector<std::string> names;
  {
    std::string all(paths), cur;
    for (char c : all) { if (c == '\n') { names.push_back(cur); cur.clear(); } else cur.push_back(c); }
    if (!cur.empty()) names.push_back(cur);
  }
  if (int(names.size()) != npaths) return fail("scatter_rows: path count mismatch");
  std::vector<uint8_t> tmp;
  for (int p = 0; p < npaths; ++p) {
    DatasetInfo* dp;
    if (!dataset_info(r, names[p], dp)) return -1;
    DatasetInfo& d = *dp;
    const uint64_t rb = d.cols * d.elem_size;
    if (rb > dst_row_stride) return fail("scatter_rows: destination rows are too short");
    for (uint64_t i = 0; i < n; ++i)
      if (rows[i] >= d.rows) return fail("row index out of range");
    bool plain_chunks = d.layout == 2 && !d.deflate && !d.shuffle && d.chunk_rows > 0 && d.btree_addr != UNDEF && load_chunk_index(r, d);
    if (plain_chunks) {
      for (size_t c = 0; c < d.chunks.size(); ++c)
        if (d.chunk_mask[c] != 0 || d.chunks[c].nbytes != d.chunk_rows * rb || !r.ok(d.chunks[c].addr, d.chunk_rows * rb)) { plain_chunks = false; break; }
    }
    if (d.layout == 1 && d.data_addr != UNDEF) {
      if (!r.ok(d.data_addr, d.rows * rb)) return fail("dataset outside the file");
      jobs.push_back({r.base + d.data_addr, static_cast<uint8_t*>(dst_bases[p]), rb, 0, {}});
    } else if (plain_chunks) {
      Job j{nullptr, static_cast<uint8_t*>(dst_bases[p]), rb, d.chunk_rows, {}};
      j.chunk_addr.assign((d.rows + d.chunk_rows - 1) / d.chunk_rows, UNDEF);
      for (const ChunkRec& c : d.chunks)
        if (c.row0 / d.chunk_rows < j.chunk_addr.size()) j.chunk_addr[c.row0 / d.chunk_rows] = c.addr;
      jobs.push_back(std::move(j));
    } else {
      tmp.resize(n * rb);
      if (read_rows_impl(r, names[p], rows, n, false, tmp.data()) != 0) return -1;
      uint8_t* dst = static_cast<uint8_t*>(dst_bases[p]);
      for (uint64_t i = 0; i < n; ++i) memcpy(dst + uint64_t(dst_pos[i]) * dst_row_stride, tmp.data() + i * rb, rb);
    }
  }
  if (jobs.empty() || n == 0) return 0;
  const uint64_t total = uint64_t(jobs.size()) * n;
  int T = nthreads < 1 ? 1 : nthreads;
  if (uint64_t(T) > total / 256 + 1) T = int(total / 256 + 1);
  auto work = [&](uint64_t lo, uint64_t hi) {
    for (uint64_t k = lo; k < hi;) {
      const Job& j = jobs[k / n];
      const uint64_t i = k % n;
      const uint64_t row = rows[i];
      // consecutive source rows (of one chunk) that land in consecutive, gap-free destination rows move as one copy
      uint64_t lim = std::min<uint64_t>(hi - k, n - i);
      const uint8_t* src;
      if (j.src != nullptr) {
        src = j.src + row * j.rb;
      } else {
        const uint64_t c = row / j.chunk_rows, in_chunk = row - c * j.chunk_rows;
        lim = std::min<uint64_t>(lim, j.chunk_rows - in_chunk);
        src = j.chunk_addr[c] == UNDEF ? nullptr : r.base + j.chunk_addr[c] + in_chunk * j.rb;
      }
      uint64_t run = 1;
      if (j.rb == dst_row_stride)
        while (run < lim && rows[i + run] == row + run && dst_pos[i + run] == dst_pos[i] + int64_t(run)) ++run;
      uint8_t* dst = j.dst + uint64_t(dst_pos[i]) * dst_row_stride;
      if (src != nullptr) memcpy(dst, src, j.rb * run); else memset(dst, 0, j.rb * run);  // unallocated chunk reads as zeros
      k += run;
    }
  };
  if (T == 1) { work(0, total); return 0; }
  std::vector<std::thread> pool;
  for (int t = 0; t < T; ++t) pool.emplace_back(work, total * t / T, total * (t + 1) / T);
  for (auto& th : pool) th.join();
  return 0;
}

int clt_h5r_read_all(void* handle, const char* path, void* out) {
  Reader& r = *static_cast<Reader*>(handle);
  std::lock_guard<std::mutex> lock(r.mu);
  return read_rows_impl(r, path, nullptr, 0, true, static_cast<uint8_t*>(out));
}

}  // extern "C"
