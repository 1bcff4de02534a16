#include "cpu_algos.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <type_traits>

#include "../core/errors.hpp"
#include "../engine/host_pool.hpp"

namespace mccl {

namespace {

// 16-bit floats are carried as raw bits and computed in fp32.
struct Half { uint16_t bits; };
struct BFloat { uint16_t bits; };

template <typename T> struct Num {
  using acc = T;
  static acc load(const T& v) { return v; }
  static T store(acc v) { return v; }
};
template <> struct Num<Half> {
  using acc = float;
  static acc load(const Half& v) { return f16_bits_to_f32(v.bits); }
  static Half store(acc v) { return Half{f32_to_f16_bits(v)}; }
};
template <> struct Num<BFloat> {
  using acc = float;
  static acc load(const BFloat& v) { return bf16_bits_to_f32(v.bits); }
  static BFloat store(acc v) { return BFloat{f32_to_bf16_bits(v)}; }
};

template <typename A> A apply(RedOp op, A a, A b) {
  switch (op) {
    case RedOp::SUM: case RedOp::AVG: return static_cast<A>(a + b);
    case RedOp::MIN: return b < a ? b : a;
    case RedOp::MAX: return b > a ? b : a;
    case RedOp::PRODUCT: return static_cast<A>(a * b);
    default: break;
  }
  if constexpr (std::is_integral<A>::value) {
    switch (op) {
      case RedOp::BAND: return static_cast<A>(a & b);
      case RedOp::BOR: return static_cast<A>(a | b);
      case RedOp::BXOR: return static_cast<A>(a ^ b);
      default: break;
    }
  }
  MCCL_CHECK_T(false, TensorError, "reduce op " << redop_name(op) << " is not defined for this dtype");
  return a;
}

// bool: SUM/MAX/BOR = or, PRODUCT/MIN/BAND = and, BXOR = xor
inline uint8_t apply_bool(RedOp op, uint8_t a, uint8_t b) {
  a = a ? 1 : 0;
  b = b ? 1 : 0;
  switch (op) {
    case RedOp::SUM: case RedOp::AVG: case RedOp::MAX: case RedOp::BOR: return a | b;
    case RedOp::PRODUCT: case RedOp::MIN: case RedOp::BAND: return a & b;
    case RedOp::BXOR: return a ^ b;
    default: return a;
  }
}

template <typename T>
void reduce_typed(RedOp op, void* dstv, const void* srcv, size_t n) {
  T* dst = static_cast<T*>(dstv);
  const T* src = static_cast<const T*>(srcv);
  using A = typename Num<T>::acc;
  // Hoist the op switch out of the hot loops for the common cases.
  if (op == RedOp::SUM || op == RedOp::AVG) {
    for (size_t i = 0; i < n; ++i) dst[i] = Num<T>::store(static_cast<A>(Num<T>::load(dst[i]) + Num<T>::load(src[i])));
  } else {
    for (size_t i = 0; i < n; ++i) dst[i] = Num<T>::store(apply<A>(op, Num<T>::load(dst[i]), Num<T>::load(src[i])));
  }
}

template <typename T>
void scale_typed(void* bufv, size_t n, double s) {
  T* buf = static_cast<T*>(bufv);
  using A = typename Num<T>::acc;
  if constexpr (std::is_integral<A>::value) {
    // Scaling integers only arises for AVG: divide by the world size exactly.
    long long div = s > 0 && s < 1 ? std::llround(1.0 / s) : 0;
    if (div > 0)
      for (size_t i = 0; i < n; ++i) buf[i] = static_cast<T>(buf[i] / static_cast<A>(div));
    else
      for (size_t i = 0; i < n; ++i) buf[i] = static_cast<T>(std::llround(static_cast<double>(buf[i]) * s));
  } else {
    A sc = static_cast<A>(s);
    for (size_t i = 0; i < n; ++i) buf[i] = Num<T>::store(static_cast<A>(Num<T>::load(buf[i]) * sc));
  }
}

template <typename T>
void reduce_scale_typed(void* dstv, const void* srcv, size_t n, double s) {
  T* dst = static_cast<T*>(dstv);
  const T* src = static_cast<const T*>(srcv);
  using A = typename Num<T>::acc;
  if constexpr (std::is_integral<A>::value) {
    reduce_typed<T>(RedOp::SUM, dstv, srcv, n);
    scale_typed<T>(dstv, n, s);
  } else {
    A sc = static_cast<A>(s);
    for (size_t i = 0; i < n; ++i)
      dst[i] = Num<T>::store(static_cast<A>((Num<T>::load(dst[i]) + Num<T>::load(src[i])) * sc));
  }
}

#define MCCL_DISPATCH_DTYPE(t, FN, ...)                                   \
  switch (t) {                                                            \
    case DType::F32: FN<float>(__VA_ARGS__); break;                       \
    case DType::F64: FN<double>(__VA_ARGS__); break;                      \
    case DType::F16: FN<Half>(__VA_ARGS__); break;                        \
    case DType::BF16: FN<BFloat>(__VA_ARGS__); break;                     \
    case DType::I8: FN<int8_t>(__VA_ARGS__); break;                       \
    case DType::I16: FN<int16_t>(__VA_ARGS__); break;                     \
    case DType::I32: FN<int32_t>(__VA_ARGS__); break;                     \
    case DType::I64: FN<int64_t>(__VA_ARGS__); break;                     \
    case DType::U8: FN<uint8_t>(__VA_ARGS__); break;                      \
    default: MCCL_CHECK_T(false, TensorError, "unsupported dtype");       \
  }

inline char* at(void* base, size_t elem_off, size_t esize) { return static_cast<char*>(base) + elem_off * esize; }
inline const char* at(const void* base, size_t elem_off, size_t esize) {
  return static_cast<const char*>(base) + elem_off * esize;
}

bool use_bf16_wire(const AllreduceArgs& a) { return a.wire == WireDtype::BF16 && a.dtype == DType::F32; }

}  // namespace

void reduce_into(DType t, RedOp op, void* dst, const void* src, size_t n) {
  if (t == DType::BOOL) {
    auto* d = static_cast<uint8_t*>(dst);
    auto* s = static_cast<const uint8_t*>(src);
    for (size_t i = 0; i < n; ++i) d[i] = apply_bool(op, d[i], s[i]);
    return;
  }
  MCCL_DISPATCH_DTYPE(t, reduce_typed, op, dst, src, n);
}

void scale_inplace(DType t, void* buf, size_t n, double s) {
  if (t == DType::BOOL) return;
  MCCL_DISPATCH_DTYPE(t, scale_typed, buf, n, s);
}

void reduce_scale(DType t, void* dst, const void* src, size_t n, double s) {
  MCCL_CHECK_T(t != DType::BOOL, TensorError, "reduce_scale is not defined for bool");
  MCCL_DISPATCH_DTYPE(t, reduce_scale_typed, dst, src, n, s);
}

void f32_to_bf16(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_bits(src[i]);
}
void bf16_to_f32(const uint16_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = bf16_bits_to_f32(src[i]);
}
void reduce_bf16_into_f32(RedOp op, float* dst, const uint16_t* src, size_t n) {
  if (op == RedOp::SUM || op == RedOp::AVG) {
    for (size_t i = 0; i < n; ++i) dst[i] += bf16_bits_to_f32(src[i]);
  } else {
    for (size_t i = 0; i < n; ++i) dst[i] = apply<float>(op, dst[i], bf16_bits_to_f32(src[i]));
  }
}
void round_f32_to_bf16_inplace(float* buf, size_t n) {
  for (size_t i = 0; i < n; ++i) buf[i] = bf16_bits_to_f32(f32_to_bf16_bits(buf[i]));
}

Algo resolve_cpu_algo(Algo requested, size_t numel, size_t bytes, int world, int64_t tree_below) {
  Algo a = requested;
  if (a == Algo::ONESHOT) a = Algo::TREE;
  if (a == Algo::NVLS) a = Algo::BUTTERFLY;
  if (a == Algo::AUTO) a = (static_cast<int64_t>(bytes) <= tree_below) ? Algo::TREE : Algo::RING;
  if (a == Algo::RING && numel < static_cast<size_t>(world)) a = Algo::TREE;
  if (a == Algo::BUTTERFLY && (world < 2 || numel < static_cast<size_t>(world))) a = Algo::TREE;
  return a;
}

void allreduce(TcpMesh& mesh, const AllreduceArgs& a, Algo algo) {
  switch (algo) {
    case Algo::RING: allreduce_ring(mesh, a); break;
    case Algo::BUTTERFLY: allreduce_butterfly(mesh, a); break;
    default: allreduce_tree(mesh, a); break;
  }
}

// ------------------------------------------------------------------ ring --
void allreduce_ring(TcpMesh& mesh, const AllreduceArgs& a) {
  const int N = mesh.world(), r = mesh.rank();
  if (N <= 1 || a.numel == 0) return;
  const size_t es = dtype_size(a.dtype);
  const bool bw = use_bf16_wire(a);
  Chunks ch(a.numel, N);
  const int next = (r + 1) % N, prev = (r - 1 + N) % N;
  const size_t wes = bw ? 2 : es;
  PooledBuffer rbuf = HostPool::staging().acquire(ch.per * wes);
  PooledBuffer sbuf = bw ? HostPool::staging().acquire(ch.per * 2) : PooledBuffer();

  auto mod = [N](int x) { return ((x % N) + N) % N; };

  for (int k = 0; k < N - 1; ++k) {
    int sc = mod(r - k), rc = mod(r - k - 1);
    const void* sp = at(a.data, ch.offset(sc), es);
    if (bw) {
      f32_to_bf16(reinterpret_cast<const float*>(sp), sbuf.as<uint16_t>(), ch.len(sc));
      sp = sbuf.data();
    }
    mesh.sendrecv(next, sp, ch.len(sc) * wes, prev, rbuf.data(), ch.len(rc) * wes);
    if (bw)
      reduce_bf16_into_f32(a.op, reinterpret_cast<float*>(at(a.data, ch.offset(rc), es)), rbuf.as<uint16_t>(),
                           ch.len(rc));
    else
      reduce_into(a.dtype, a.op, at(a.data, ch.offset(rc), es), rbuf.data(), ch.len(rc));
  }
  // Rank r now owns the fully reduced chunk (r+1) mod N.
  const int own = mod(r + 1);
  if (bw) round_f32_to_bf16_inplace(reinterpret_cast<float*>(at(a.data, ch.offset(own), es)), ch.len(own));
  for (int k = 0; k < N - 1; ++k) {
    int sc = mod(r + 1 - k), rc = mod(r - k);
    if (bw) {
      f32_to_bf16(reinterpret_cast<const float*>(at(a.data, ch.offset(sc), es)), sbuf.as<uint16_t>(), ch.len(sc));
      mesh.sendrecv(next, sbuf.data(), ch.len(sc) * 2, prev, rbuf.data(), ch.len(rc) * 2);
      bf16_to_f32(rbuf.as<uint16_t>(), reinterpret_cast<float*>(at(a.data, ch.offset(rc), es)), ch.len(rc));
    } else {
      mesh.sendrecv(next, at(a.data, ch.offset(sc), es), ch.len(sc) * es, prev, at(a.data, ch.offset(rc), es),
                    ch.len(rc) * es);
    }
  }
  if (a.op == RedOp::AVG) scale_inplace(a.dtype, a.data, a.numel, 1.0 / N);
}

// ------------------------------------------------------------------ tree --
void allreduce_tree(TcpMesh& mesh, const AllreduceArgs& a) {
  const int N = mesh.world(), r = mesh.rank();
  if (N <= 1 || a.numel == 0) return;
  const size_t es = dtype_size(a.dtype);
  const bool bw = use_bf16_wire(a);
  const size_t wes = bw ? 2 : es;
  PooledBuffer stage = HostPool::staging().acquire(a.numel * wes);

  // reduce towards rank 0
  for (int mask = 1; mask < N; mask <<= 1) {
    if (r & mask) {
      const void* sp = a.data;
      if (bw) {
        f32_to_bf16(static_cast<const float*>(a.data), stage.as<uint16_t>(), a.numel);
        sp = stage.data();
      }
      mesh.send(r - mask, sp, a.numel * wes);
      break;
    }
    if (r + mask < N) {
      mesh.recv(r + mask, stage.data(), a.numel * wes);
      if (bw)
        reduce_bf16_into_f32(a.op, static_cast<float*>(a.data), stage.as<uint16_t>(), a.numel);
      else
        reduce_into(a.dtype, a.op, a.data, stage.data(), a.numel);
    }
  }
  // broadcast from rank 0
  if (bw) {
    if (r == 0) f32_to_bf16(static_cast<const float*>(a.data), stage.as<uint16_t>(), a.numel);
    broadcast(mesh, stage.data(), a.numel * 2, 0);
    bf16_to_f32(stage.as<uint16_t>(), static_cast<float*>(a.data), a.numel);
  } else {
    broadcast(mesh, a.data, a.numel * es, 0);
  }
  if (a.op == RedOp::AVG) scale_inplace(a.dtype, a.data, a.numel, 1.0 / N);
}

// ------------------------------------------------------------- butterfly --
void allreduce_butterfly(TcpMesh& mesh, const AllreduceArgs& a) {
  const int N = mesh.world(), r = mesh.rank();
  if (N <= 1 || a.numel == 0) return;
  const size_t es = dtype_size(a.dtype);
  const bool bw = use_bf16_wire(a);
  const size_t wes = bw ? 2 : es;
  Chunks ch(a.numel, N);
  const size_t mylen = ch.len(r);

  // Phase 1: send chunk p to peer p, receive every peer's copy of chunk r.
  PooledBuffer rstage = HostPool::staging().acquire(static_cast<size_t>(N - 1) * ch.per * wes);
  PooledBuffer sstage = bw ? HostPool::staging().acquire(a.numel * 2) : PooledBuffer();
  if (bw) f32_to_bf16(static_cast<const float*>(a.data), sstage.as<uint16_t>(), a.numel);
  std::vector<IoSpan> sends, recvs;
  int slot = 0;
  for (int p = 0; p < N; ++p) {
    if (p == r) continue;
    void* sp = bw ? static_cast<void*>(sstage.as<uint16_t>() + ch.offset(p)) : at(a.data, ch.offset(p), es);
    sends.push_back({p, sp, ch.len(p) * wes});
    recvs.push_back({p, rstage.as<char>() + static_cast<size_t>(slot) * ch.per * wes, mylen * wes});
    ++slot;
  }
  mesh.exchange(sends, recvs);
  // Local reduce in ascending peer order.
  char* mine = at(a.data, ch.offset(r), es);
  for (int s = 0; s < N - 1; ++s) {
    const char* src = rstage.as<char>() + static_cast<size_t>(s) * ch.per * wes;
    if (bw)
      reduce_bf16_into_f32(a.op, reinterpret_cast<float*>(mine), reinterpret_cast<const uint16_t*>(src), mylen);
    else
      reduce_into(a.dtype, a.op, mine, src, mylen);
  }
  if (a.op == RedOp::AVG) scale_inplace(a.dtype, mine, mylen, 1.0 / N);
  if (bw) round_f32_to_bf16_inplace(reinterpret_cast<float*>(mine), mylen);

  // Phase 2: allgather of the reduced chunks.
  sends.clear();
  recvs.clear();
  if (bw) {
    f32_to_bf16(reinterpret_cast<const float*>(mine), sstage.as<uint16_t>() + ch.offset(r), mylen);
    PooledBuffer gstage = HostPool::staging().acquire(a.numel * 2);
    for (int p = 0; p < N; ++p) {
      if (p == r) continue;
      sends.push_back({p, sstage.as<uint16_t>() + ch.offset(r), mylen * 2});
      recvs.push_back({p, gstage.as<uint16_t>() + ch.offset(p), ch.len(p) * 2});
    }
    mesh.exchange(sends, recvs);
    for (int p = 0; p < N; ++p)
      if (p != r)
        bf16_to_f32(gstage.as<uint16_t>() + ch.offset(p), reinterpret_cast<float*>(at(a.data, ch.offset(p), es)),
                    ch.len(p));
  } else {
    for (int p = 0; p < N; ++p) {
      if (p == r) continue;
      sends.push_back({p, mine, mylen * es});
      recvs.push_back({p, at(a.data, ch.offset(p), es), ch.len(p) * es});
    }
    mesh.exchange(sends, recvs);
  }
}

// ------------------------------------------------------- other collectives --
void broadcast(TcpMesh& mesh, void* data, size_t nbytes, int root) {
  const int N = mesh.world();
  if (N <= 1 || nbytes == 0) return;
  const int vr = (mesh.rank() - root + N) % N;  // rank relative to the root
  int mask = 1;
  while (mask < N) {
    if (vr & mask) {
      mesh.recv((vr - mask + root) % N, data, nbytes);
      break;
    }
    mask <<= 1;
  }
  mask >>= 1;
  while (mask > 0) {
    if (vr + mask < N) mesh.send((vr + mask + root) % N, data, nbytes);
    mask >>= 1;
  }
}

void reduce(TcpMesh& mesh, void* data, size_t numel, DType t, RedOp op, int root) {
  const int N = mesh.world();
  if (N <= 1 || numel == 0) return;
  const size_t es = dtype_size(t);
  const int vr = (mesh.rank() - root + N) % N;
  PooledBuffer stage = HostPool::staging().acquire(numel * es);
  for (int mask = 1; mask < N; mask <<= 1) {
    if (vr & mask) {
      mesh.send((vr - mask + root) % N, data, numel * es);
      break;
    }
    if (vr + mask < N) {
      mesh.recv((vr + mask + root) % N, stage.data(), numel * es);
      reduce_into(t, op, data, stage.data(), numel);
    }
  }
  if (op == RedOp::AVG && vr == 0) scale_inplace(t, data, numel, 1.0 / N);
}

void allgather(TcpMesh& mesh, const void* in, void* out, size_t nbytes) {
  const int N = mesh.world(), r = mesh.rank();
  char* o = static_cast<char*>(out);
  if (o + static_cast<size_t>(r) * nbytes != in) std::memmove(o + static_cast<size_t>(r) * nbytes, in, nbytes);
  if (N <= 1 || nbytes == 0) return;
  std::vector<IoSpan> sends, recvs;
  for (int p = 0; p < N; ++p) {
    if (p == r) continue;
    sends.push_back({p, o + static_cast<size_t>(r) * nbytes, nbytes});
    recvs.push_back({p, o + static_cast<size_t>(p) * nbytes, nbytes});
  }
  mesh.exchange(sends, recvs);
}

void reduce_scatter(TcpMesh& mesh, const void* in, void* out, size_t numel, DType t, RedOp op) {
  const int N = mesh.world(), r = mesh.rank();
  const size_t es = dtype_size(t), cb = numel * es;
  const char* i = static_cast<const char*>(in);
  if (N <= 1) {
    if (out != in) std::memmove(out, in, cb);
    return;
  }
  PooledBuffer stage = HostPool::staging().acquire(static_cast<size_t>(N - 1) * cb);
  std::vector<IoSpan> sends, recvs;
  int slot = 0;
  for (int p = 0; p < N; ++p) {
    if (p == r) continue;
    sends.push_back({p, const_cast<char*>(i) + static_cast<size_t>(p) * cb, cb});
    recvs.push_back({p, stage.as<char>() + static_cast<size_t>(slot++) * cb, cb});
  }
  mesh.exchange(sends, recvs);
  // Seed with the own slice only after the exchange: out may alias a slice of in.
  if (out != i + static_cast<size_t>(r) * cb) std::memmove(out, i + static_cast<size_t>(r) * cb, cb);
  for (int s = 0; s < N - 1; ++s) reduce_into(t, op, out, stage.as<char>() + static_cast<size_t>(s) * cb, numel);
  if (op == RedOp::AVG) scale_inplace(t, out, numel, 1.0 / N);
}

void alltoallv(TcpMesh& mesh, const void* in, const std::vector<size_t>& in_off, const std::vector<size_t>& in_len,
               void* out, const std::vector<size_t>& out_off, const std::vector<size_t>& out_len) {
  const int N = mesh.world(), r = mesh.rank();
  const char* i = static_cast<const char*>(in);
  char* o = static_cast<char*>(out);
  MCCL_CHECK(in_len[r] == out_len[r], "alltoall: self split mismatch (" << in_len[r] << " vs " << out_len[r] << ")");
  if (in_len[r]) std::memmove(o + out_off[r], i + in_off[r], in_len[r]);
  std::vector<IoSpan> sends, recvs;
  for (int p = 0; p < N; ++p) {
    if (p == r) continue;
    if (in_len[p]) sends.push_back({p, const_cast<char*>(i) + in_off[p], in_len[p]});
    if (out_len[p]) recvs.push_back({p, o + out_off[p], out_len[p]});
  }
  mesh.exchange(sends, recvs);
}

void gather(TcpMesh& mesh, const void* in, void* out, size_t nbytes, int root) {
  const int N = mesh.world(), r = mesh.rank();
  if (r == root) {
    char* o = static_cast<char*>(out);
    std::memmove(o + static_cast<size_t>(r) * nbytes, in, nbytes);
    std::vector<IoSpan> recvs;
    for (int p = 0; p < N; ++p)
      if (p != r) recvs.push_back({p, o + static_cast<size_t>(p) * nbytes, nbytes});
    mesh.exchange({}, recvs);
  } else {
    mesh.send(root, in, nbytes);
  }
}

void scatter(TcpMesh& mesh, const void* in, void* out, size_t nbytes, int root) {
  const int N = mesh.world(), r = mesh.rank();
  if (r == root) {
    const char* i = static_cast<const char*>(in);
    std::vector<IoSpan> sends;
    for (int p = 0; p < N; ++p)
      if (p != r) sends.push_back({p, const_cast<char*>(i) + static_cast<size_t>(p) * nbytes, nbytes});
    mesh.exchange(sends, {});
    std::memmove(out, i + static_cast<size_t>(r) * nbytes, nbytes);
  } else {
    mesh.recv(root, out, nbytes);
  }
}

namespace {
#pragma pack(push, 1)
struct P2PHeader {
  int32_t tag;
  int64_t nbytes;
};
#pragma pack(pop)
}  // namespace

void send_tagged(TcpMesh& mesh, int dst, const void* data, size_t nbytes, int tag) {
  P2PHeader h{tag, static_cast<int64_t>(nbytes)};
  std::vector<IoSpan> sends{{dst, &h, sizeof(h)}};
  if (nbytes) sends.push_back({dst, const_cast<void*>(data), nbytes});
  mesh.exchange(sends, {});
}

void recv_tagged(TcpMesh& mesh, int src, void* data, size_t nbytes, int tag) {
  P2PHeader h{};
  mesh.recv(src, &h, sizeof(h));
  MCCL_CHECK_T(h.nbytes == static_cast<int64_t>(nbytes), ProtocolError,
               "recv: size mismatch from rank " << src << ": sender has " << h.nbytes << " bytes, receiver expects "
                                                << nbytes);
  if (nbytes) mesh.recv(src, data, nbytes);
  MCCL_CHECK_T(tag < 0 || h.tag == tag, ProtocolError,
               "recv: tag mismatch from rank " << src << ": got " << h.tag << ", expected " << tag);
}

}  // namespace mccl
