// xoroshiro128+ : parallel state creation with jump-ahead, and fused bulk draws.
//
// State creation.  The reference builds the states on the CPU as a serial
// chain, state[i] = jump(state[i-1]) with 128 generator steps per jump
// (numba/cuda/random.py:242-257), then copies them to the device.  Here every
// thread computes its states directly:
//
//   * the generator step is linear over GF(2), so jump is a 128x128 bit matrix J
//     and state[i] = J^i v (v = SplitMix64 of the seed, random.py:63-85);
//   * J is annihilated by a degree-128 polynomial P (found once per process by
//     solving u_128 = sum_j P_j u_j over GF(2) on a probe sequence u_j = J^j v0,
//     then re-checked on a second probe), hence
//         J^i v = sum_j c_j u_j   with  c(y) = y^i mod P(y),  u_j = J^j v;
//   * the host computes the 128 seed-dependent basis states u_j with the serial
//     recipe (16 k generator steps) and passes them as a kernel parameter;
//   * a thread owning states [first, first+L) gets y^(start+first) mod P as a
//     product of per-byte table entries Y[l][b] = y^(b*256^l) (seed-independent
//     table in device memory), then alternates "combine basis states under the
//     128-bit mask c" and "c <- c*y mod P" (one shift and one conditional xor).
//
// Bulk draws.  One lane owns one generator, keeps (s0, s1) in registers for all
// its draws and writes the state back once (the reference reloads and stores
// the state on every draw, random.py:97-115).  Each warp stages a 32-generator
// x 32-value block in shared memory and flushes it row by row so that every
// global store instruction covers whole 128-byte lines of the [n, count] output.
#include <cmath>
#include <cstring>
#include <mutex>

#include "../../include/b2k_xoroshiro128p.cuh"
#include "b2k_internal.cuh"

namespace {

// ---- host-side restatement of the generator (random.py:63-142) --------------
struct State { uint64_t s0, s1; };

inline uint64_t rotl_h(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

inline State seed_state(uint64_t seed) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return State{z, z};
}
inline void step_h(State &s) {
    uint64_t a = s.s0, b = s.s1 ^ s.s0;
    s.s0 = rotl_h(a, 55) ^ b ^ (b << 14);
    s.s1 = rotl_h(b, 36);
}
inline void jump_h(State &s) {
    static const uint64_t kJump[2] = {0xBEAC0467EBA5FACBull, 0xD86B048B86AA9922ull};
    uint64_t a0 = 0, a1 = 0;
    for (int w = 0; w < 2; ++w)
        for (int b = 0; b < 64; ++b) {
            if ((kJump[w] >> b) & 1ull) { a0 ^= s.s0; a1 ^= s.s1; }
            step_h(s);
        }
    s.s0 = a0;
    s.s1 = a1;
}

// ---- GF(2)[y] / P(y) ------------------------------------------------------------
struct Poly { uint64_t lo, hi; };  // coefficient of y^k is bit k

struct RingConstants {
    bool ready = false;
    bool valid = false;
    Poly p_low{};                  // P(y) = y^128 + p_low(y)
    Poly ytab[8][256];             // ytab[l][b] = y^(b * 256^l) mod P
};
RingConstants g_ring;
std::mutex g_ring_mutex;

inline Poly times_y(Poly a, const Poly &p_low) {
    const bool carry = (a.hi >> 63) != 0;
    a.hi = (a.hi << 1) | (a.lo >> 63);
    a.lo <<= 1;
    if (carry) { a.lo ^= p_low.lo; a.hi ^= p_low.hi; }
    return a;
}
inline Poly mulmod_h(const Poly &a, const Poly &b, const Poly &p_low) {
    Poly r{0, 0};
    for (int i = 127; i >= 0; --i) {
        r = times_y(r, p_low);
        const uint64_t bit = (i < 64) ? (a.lo >> i) & 1ull : (a.hi >> (i - 64)) & 1ull;
        if (bit) { r.lo ^= b.lo; r.hi ^= b.hi; }
    }
    return r;
}

// Solve sum_j c_j u_j = u_128 over GF(2) for the coefficient mask c.
bool solve_recurrence(const State *u /* 129 states */, Poly *out) {
    // rows = the 128 state bits; columns 0..127 = u_j, column 128 = right-hand side
    struct Row { uint64_t w[3]; };
    Row rows[128];
    for (int bit = 0; bit < 128; ++bit) {
        Row r{{0, 0, 0}};
        for (int j = 0; j <= 128; ++j) {
            const uint64_t word = bit < 64 ? u[j].s0 : u[j].s1;
            if ((word >> (bit & 63)) & 1ull) r.w[j >> 6] |= 1ull << (j & 63);
        }
        rows[bit] = r;
    }
    int pivot_row_of_col[128];
    int next_row = 0;
    for (int col = 0; col < 128; ++col) {
        int found = -1;
        for (int r = next_row; r < 128; ++r)
            if ((rows[r].w[col >> 6] >> (col & 63)) & 1ull) { found = r; break; }
        if (found < 0) return false;  // basis not of full rank
        Row tmp = rows[found]; rows[found] = rows[next_row]; rows[next_row] = tmp;
        for (int r = 0; r < 128; ++r)
            if (r != next_row && ((rows[r].w[col >> 6] >> (col & 63)) & 1ull))
                for (int k = 0; k < 3; ++k) rows[r].w[k] ^= rows[next_row].w[k];
        pivot_row_of_col[col] = next_row++;
    }
    Poly c{0, 0};
    for (int col = 0; col < 128; ++col)
        if (rows[pivot_row_of_col[col]].w[2] & 1ull) {
            if (col < 64) c.lo |= 1ull << col; else c.hi |= 1ull << (col - 64);
        }
    *out = c;
    return true;
}

void basis_states(uint64_t seed, State *u, int count) {
    u[0] = seed_state(seed);
    for (int j = 1; j < count; ++j) { u[j] = u[j - 1]; jump_h(u[j]); }
}

const RingConstants &ring() {
    std::lock_guard<std::mutex> lock(g_ring_mutex);
    if (g_ring.ready) return g_ring;
    g_ring.ready = true;
    State u[129];
    basis_states(0x243F6A8885A308D3ull, u, 129);
    Poly p{};
    if (!solve_recurrence(u, &p)) return g_ring;
    // independent check on another sequence: u_128 must equal the masked xor
    basis_states(0x13198A2E03707344ull, u, 129);
    uint64_t x0 = 0, x1 = 0;
    for (int j = 0; j < 128; ++j) {
        const uint64_t bit = j < 64 ? (p.lo >> j) & 1ull : (p.hi >> (j - 64)) & 1ull;
        if (bit) { x0 ^= u[j].s0; x1 ^= u[j].s1; }
    }
    if (x0 != u[128].s0 || x1 != u[128].s1) return g_ring;
    g_ring.p_low = p;
    Poly base{2, 0};  // y
    for (int l = 0; l < 8; ++l) {
        g_ring.ytab[l][0] = Poly{1, 0};
        g_ring.ytab[l][1] = base;
        for (int b = 2; b < 256; ++b) g_ring.ytab[l][b] = mulmod_h(g_ring.ytab[l][b - 1], base, p);
        base = mulmod_h(g_ring.ytab[l][255], base, p);
    }
    g_ring.valid = true;
    return g_ring;
}

constexpr int64_t kTablesBytes = 8 * 256 * 16;

// ---- device: state creation -------------------------------------------------------
struct Basis { uint32_t w[128][4]; };  // u_j as four little-endian 32-bit words

struct Poly4 { uint32_t w[4]; };

__device__ __forceinline__ void times_y_d(Poly4 &a, const Poly4 &p_low) {
    const uint32_t carry = static_cast<uint32_t>(static_cast<int32_t>(a.w[3]) >> 31);  // 0 or ~0
    a.w[3] = __funnelshift_l(a.w[2], a.w[3], 1);
    a.w[2] = __funnelshift_l(a.w[1], a.w[2], 1);
    a.w[1] = __funnelshift_l(a.w[0], a.w[1], 1);
    a.w[0] <<= 1;
#pragma unroll
    for (int k = 0; k < 4; ++k) a.w[k] ^= carry & p_low.w[k];
}

__device__ __forceinline__ Poly4 mulmod_d(const Poly4 &a, const Poly4 &b, const Poly4 &p_low) {
    Poly4 r{{0, 0, 0, 0}};
    for (int word = 3; word >= 0; --word) {
        const uint32_t aw = a.w[word];
        for (int bit = 31; bit >= 0; --bit) {
            times_y_d(r, p_low);
            const uint32_t m = static_cast<uint32_t>(static_cast<int32_t>(aw << (31 - bit)) >> 31);
#pragma unroll
            for (int k = 0; k < 4; ++k) r.w[k] ^= m & b.w[k];
        }
    }
    return r;
}

__global__ void __launch_bounds__(256)
xoro_init_kernel(uint4 *__restrict__ states, int64_t n, uint64_t start, int per_thread,
                 const uint4 *__restrict__ ytab, const __grid_constant__ Basis basis,
                 const Poly4 p_low) {
    const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t first = t * per_thread;
    if (first >= n) return;

    // c(y) = y^(start + first) mod P, one table entry per non-zero exponent byte
    const uint64_t e = start + static_cast<uint64_t>(first);
    Poly4 c{{1, 0, 0, 0}};
    bool have = false;
    for (int l = 0; l < 8; ++l) {
        const uint32_t b = static_cast<uint32_t>(e >> (8 * l)) & 0xFFu;
        if (b == 0) continue;
        const uint4 raw = __ldg(ytab + l * 256 + b);
        const Poly4 f{{raw.x, raw.y, raw.z, raw.w}};
        c = have ? mulmod_d(c, f, p_low) : f;
        have = true;
    }

    const int64_t last = (first + per_thread < n) ? first + per_thread : n;
    for (int64_t i = first; i < last; ++i) {
        uint32_t s0 = 0, s1 = 0, s2 = 0, s3 = 0;
#pragma unroll
        for (int j = 0; j < 128; ++j) {
            const uint32_t m =
                static_cast<uint32_t>(static_cast<int32_t>(c.w[j >> 5] << (31 - (j & 31))) >> 31);
            s0 ^= m & basis.w[j][0];
            s1 ^= m & basis.w[j][1];
            s2 ^= m & basis.w[j][2];
            s3 ^= m & basis.w[j][3];
        }
        states[i] = make_uint4(s0, s1, s2, s3);
        times_y_d(c, p_low);
    }
}

// Large arrays: the 128-term masked xor above keeps the integer pipe busy (about
// 5 instructions per basis state).  This variant first expands the 128 basis
// states into byte-indexed tables in shared memory, T[v][p] = xor of the basis
// states selected by byte value v at byte position p of the mask (64 KB per CTA,
// built once per CTA), after which a state costs 16 128-bit shared loads and 16
// three-input xors per word.
//
// Bank conflicts: a 128-bit shared load is served a quarter-warp at a time, and
// eight 16-byte entries collide unless they sit in eight different 16-byte slots
// of the 128-byte bank row.  The byte values v are random, so the slot must not
// depend on v: entries are laid out [v][p] (slot = p mod 8) and lane l walks the
// byte positions in the rotated order p = (t + l) mod 16, t = 0..15, so the eight
// lanes of a quarter-warp always read eight different slots.  The rotation is
// applied to the mask once per state (a 128-bit byte rotate by l mod 16), after
// which byte t of the rotated mask is extracted with a constant selector.
//
// Every thread owns ONE contiguous run of `per_thread` states (an even number), so
// y^index is built once per thread and then advanced by single steps, and states
// leave in pairs as 32-byte stores when `states` is 32-byte aligned.
constexpr int kTableBytes = 16 * 256 * 16;

__device__ __forceinline__ void store_state_pair(uint4 *dst, const uint4 &a, const uint4 &b) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst), "r"(a.x), "r"(a.y), "r"(a.z),
                 "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}

template <int T>
__device__ __forceinline__ void table_lookup(const unsigned char *tb, const uint32_t (&w)[4], uint32_t r16,
                                             uint32_t &s0, uint32_t &s1, uint32_t &s2, uint32_t &s3) {
    // byte (T & 3) of word T / 4, moved to bits 8..15: the byte offset v * 256
    constexpr uint32_t kSel = 0x4404u | ((T & 3) << 4);
    const uint32_t voff = __byte_perm(w[T >> 2], 0u, kSel);
    const uint32_t poff = (r16 + 16u * T) & 0xF0u;
    const uint4 e = *reinterpret_cast<const uint4 *>(tb + voff + poff);
    s0 ^= e.x;
    s1 ^= e.y;
    s2 ^= e.z;
    s3 ^= e.w;
}

__device__ __forceinline__ uint4 state_from_mask(const unsigned char *tb, const Poly4 &c, uint32_t r) {
    // rotate the 16 mask bytes down by r: byte t of w = byte (t + r) mod 16 of c
    const bool r4 = (r & 4u) != 0, r8 = (r & 8u) != 0;
    const uint32_t sh = (r & 3u) * 8u;
    const uint32_t y0 = r4 ? c.w[1] : c.w[0], y1 = r4 ? c.w[2] : c.w[1];
    const uint32_t y2 = r4 ? c.w[3] : c.w[2], y3 = r4 ? c.w[0] : c.w[3];
    const uint32_t x0 = r8 ? y2 : y0, x1 = r8 ? y3 : y1, x2 = r8 ? y0 : y2, x3 = r8 ? y1 : y3;
    const uint32_t w[4] = {__funnelshift_r(x0, x1, sh), __funnelshift_r(x1, x2, sh), __funnelshift_r(x2, x3, sh),
                           __funnelshift_r(x3, x0, sh)};
    const uint32_t r16 = r * 16u;
    uint32_t s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    table_lookup<0>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<1>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<2>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<3>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<4>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<5>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<6>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<7>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<8>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<9>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<10>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<11>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<12>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<13>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<14>(tb, w, r16, s0, s1, s2, s3);
    table_lookup<15>(tb, w, r16, s0, s1, s2, s3);
    return make_uint4(s0, s1, s2, s3);
}

__global__ void __launch_bounds__(256)
xoro_init_table_kernel(uint4 *__restrict__ states, int64_t n, uint64_t start, int per_thread, int wide_stores,
                       const uint4 *__restrict__ ytab, const __grid_constant__ Basis basis,
                       const Poly4 p_low) {
    extern __shared__ uint4 table[];  // [256][16]
    {
        const uint32_t v = threadIdx.x;  // byte value owned by this thread
#pragma unroll
        for (int p = 0; p < 16; ++p) {
            uint32_t t0 = 0, t1 = 0, t2 = 0, t3 = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t m = static_cast<uint32_t>(static_cast<int32_t>(v << (31 - i)) >> 31);
                t0 ^= m & basis.w[8 * p + i][0];
                t1 ^= m & basis.w[8 * p + i][1];
                t2 ^= m & basis.w[8 * p + i][2];
                t3 ^= m & basis.w[8 * p + i][3];
            }
            table[v * 16 + p] = make_uint4(t0, t1, t2, t3);
        }
    }
    __syncthreads();

    const unsigned char *tb = reinterpret_cast<const unsigned char *>(table);
    const uint32_t r = threadIdx.x & 15u;
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * per_thread;
    if (first >= n) return;
    const uint64_t e = start + static_cast<uint64_t>(first);
    Poly4 c{{1, 0, 0, 0}};
    bool have = false;
    for (int l = 0; l < 8; ++l) {
        const uint32_t b = static_cast<uint32_t>(e >> (8 * l)) & 0xFFu;
        if (b == 0) continue;
        const uint4 raw = __ldg(ytab + l * 256 + b);
        const Poly4 f{{raw.x, raw.y, raw.z, raw.w}};
        c = have ? mulmod_d(c, f, p_low) : f;
        have = true;
    }
    const int64_t last = (first + per_thread < n) ? first + per_thread : n;
    int64_t i = first;
    if (wide_stores) {  // `first` is even and `states` 32-byte aligned
        for (; i + 2 <= last; i += 2) {
            const uint4 a = state_from_mask(tb, c, r);
            times_y_d(c, p_low);
            const uint4 b = state_from_mask(tb, c, r);
            times_y_d(c, p_low);
            store_state_pair(states + i, a, b);
        }
    }
    for (; i < last; ++i) {
        states[i] = state_from_mask(tb, c, r);
        times_y_d(c, p_low);
    }
}

// ---- device: draws ------------------------------------------------------------------
// The generator arithmetic lives in include/b2k_xoroshiro128p.cuh so that user
// CUDA C++ kernels and this library draw from the same code.

struct Segment {
    void *out;
    int64_t count;
    int draw;
};

constexpr int kFillWarps = 8;
constexpr int kStageBytes = 32 * 128;  // 32 rows of 128 bytes per warp

template <typename T, int DRAW>
__device__ __forceinline__ T draw_one(uint64_t &s0, uint64_t &s1) {
    xoroshiro128p_generator g(s0, s1);
    T r;
    if constexpr (DRAW == B2K_UNIFORM_F32) r = g.uniform_float32();
    else if constexpr (DRAW == B2K_UNIFORM_F64) r = g.uniform_float64();
    else if constexpr (DRAW == B2K_NORMAL_F32) r = g.normal_float32();
    else r = g.normal_float64();
    s0 = g.s0;
    s1 = g.s1;
    return r;
}

// One segment for the 32 generators [base, base+32) of this warp.
//
// Every lane draws a chunk of 128 bytes (32 f32 / 16 f64 values) into its own row of
// the warp's staging tile, 16 bytes at a time, then the warp writes the tile out
// row-wise.  Rows are 128 bytes with the 16-byte pieces XOR-swizzled by the row
// number (piece p of row r sits at piece p ^ (r & 7)), so both the lanes' 128-bit
// stores (eight rows, one piece each per quarter-warp) and the 128-bit loads of the
// flush (one row, eight pieces per quarter-warp) are free of bank conflicts.  Full
// tiles whose output rows are 16-byte aligned leave as 128-bit stores, four rows of
// 128 bytes per instruction; ragged tiles (last generators, last columns, odd
// counts) leave one row of scalars per instruction.
template <typename T>
__device__ __forceinline__ T *stage_slot(unsigned char *stage, int row, int col) {
    constexpr int PER = 16 / sizeof(T);
    return reinterpret_cast<T *>(stage + row * 128 + (((col / PER) ^ (row & 7)) << 4)) + (col % PER);
}

template <typename T, int DRAW, int UNROLL>
__device__ __forceinline__ void fill_segment(uint64_t &s0, uint64_t &s1, bool live, int64_t base,
                                             int64_t n, const Segment &seg, void *stage_ptr) {
    constexpr int CHUNK = 128 / sizeof(T);
    constexpr int ROWS_PER_STORE = 32 / CHUNK;
    constexpr int PER = 16 / sizeof(T);             // items in one 128-bit piece
    unsigned char *stage = static_cast<unsigned char *>(stage_ptr);
    T *out = static_cast<T *>(seg.out);
    const int lane = threadIdx.x & 31;
    const bool rows_full = base + 32 <= n;
    const bool vector_ok = rows_full && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0) &&
                           ((seg.count * sizeof(T)) % 16 == 0);
    for (int64_t c0 = 0; c0 < seg.count; c0 += CHUNK) {
        const int m = (seg.count - c0 < CHUNK) ? static_cast<int>(seg.count - c0) : CHUNK;
        if (live) {
            if (m == CHUNK) {
                // uniforms are short integer chains: unroll deep to overlap generators;
                // normals are long libdevice chains: unroll little to keep registers free
                constexpr int U = (DRAW == B2K_UNIFORM_F32 || DRAW == B2K_UNIFORM_F64) ? 16 : UNROLL;
                constexpr int PIECES_UNROLLED = U / PER > 0 ? U / PER : 1;
                unsigned char *row = stage + lane * 128;
                const int swizzle = (lane & 7) << 4;
#pragma unroll PIECES_UNROLLED
                for (int p = 0; p < 8; ++p) {
                    union {
                        uint4 raw;
                        T v[PER];
                    } piece;
#pragma unroll
                    for (int k = 0; k < PER; ++k) piece.v[k] = draw_one<T, DRAW>(s0, s1);
                    *reinterpret_cast<uint4 *>(row + ((p << 4) ^ swizzle)) = piece.raw;
                }
            } else {
                for (int i = 0; i < m; ++i) *stage_slot<T>(stage, lane, i) = draw_one<T, DRAW>(s0, s1);
            }
        }
        __syncwarp();
        if (vector_ok && m == CHUNK) {
            // lane -> (row within a group of four, 16-byte piece of that row)
            const int sub = lane >> 3, piece = lane & 7;
            T *dst = out + (base + sub) * seg.count + c0 + piece * PER;
            const int64_t dst_step = 4 * seg.count;
#pragma unroll
            for (int r = 0; r < 32; r += 4) {
                const int row = r + sub;
                const uint4 v = *reinterpret_cast<const uint4 *>(stage + row * 128 + ((piece ^ (row & 7)) << 4));
                __stcs(reinterpret_cast<uint4 *>(dst), v);
                dst += dst_step;
            }
        } else {
            const int col = lane % CHUNK;
            const int sub = lane / CHUNK;
            if (col < m) {
                T *dst = out + (base + sub) * seg.count + c0 + col;
                const int64_t dst_step = static_cast<int64_t>(ROWS_PER_STORE) * seg.count;
                const int64_t rows_here = n - base - sub;  // rows this lane may still write
                for (int r = 0; r < 32 && r < rows_here; r += ROWS_PER_STORE) {
                    *dst = *stage_slot<T>(stage, r + sub, col);
                    dst += dst_step;
                }
            }
        }
        __syncwarp();
    }
}

template <int UNROLL>
__device__ __forceinline__ void run_segment(uint64_t &s0, uint64_t &s1, bool live, int64_t base,
                                            int64_t n, const Segment &seg, void *stage) {
    if (seg.count <= 0) return;
    switch (seg.draw) {  // uniform across the grid
    case B2K_UNIFORM_F32: fill_segment<float, B2K_UNIFORM_F32, UNROLL>(s0, s1, live, base, n, seg, stage); break;
    case B2K_UNIFORM_F64: fill_segment<double, B2K_UNIFORM_F64, UNROLL>(s0, s1, live, base, n, seg, stage); break;
    case B2K_NORMAL_F32: fill_segment<float, B2K_NORMAL_F32, UNROLL>(s0, s1, live, base, n, seg, stage); break;
    default: fill_segment<double, B2K_NORMAL_F64, UNROLL>(s0, s1, live, base, n, seg, stage); break;
    }
}

template <int MINBLOCKS, int UNROLL>
__global__ void __launch_bounds__(kFillWarps * 32, MINBLOCKS)
xoro_fill_kernel(ulonglong2 *__restrict__ states, int64_t n, Segment seg0, Segment seg1) {
    __shared__ __align__(128) unsigned char stage_all[kFillWarps][kStageBytes];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    void *stage = stage_all[warp];
    const int64_t groups = (n + 31) / 32;
    for (int64_t grp = static_cast<int64_t>(blockIdx.x) * kFillWarps + warp; grp < groups;
         grp += static_cast<int64_t>(gridDim.x) * kFillWarps) {
        const int64_t base = grp * 32;
        const int64_t g = base + lane;
        const bool live = g < n;
        uint64_t s0 = 0, s1 = 0;
        if (live) {
            const ulonglong2 s = states[g];
            s0 = s.x;
            s1 = s.y;
        }
        run_segment<UNROLL>(s0, s1, live, base, n, seg0, stage);
        run_segment<UNROLL>(s0, s1, live, base, n, seg1, stage);
        if (live) states[g] = make_ulonglong2(s0, s1);
    }
}

size_t draw_size(int draw) {
    switch (draw) {
    case B2K_UNIFORM_F32: case B2K_NORMAL_F32: return 4;
    case B2K_UNIFORM_F64: case B2K_NORMAL_F64: return 8;
    default: return 0;
    }
}

}  // namespace

extern "C" {

int64_t b2k_xoroshiro128p_tables_bytes(void) { return kTablesBytes; }

int b2k_xoroshiro128p_build_tables(void *tables_dev, int64_t tables_bytes, void *stream) {
    B2K_RANGE("b2k_xoroshiro128p_build_tables");
    if (!tables_dev || tables_bytes < kTablesBytes)
        return b2k::fail(B2K_ERR_SCRATCH, "b2k_xoroshiro128p_build_tables: %lld bytes required",
                         (long long)kTablesBytes);
    const RingConstants &rc = ring();
    if (!rc.valid)
        return b2k::fail(B2K_ERR_UNSUPPORTED, "xoroshiro128p: jump recurrence self-check failed");
    // the source is static storage that is never modified after construction
    return b2k::check_cuda(cudaMemcpyAsync(tables_dev, rc.ytab, kTablesBytes, cudaMemcpyHostToDevice,
                                           b2k::as_stream(stream)),
                           "b2k_xoroshiro128p_build_tables copy");
}

int b2k_xoroshiro128p_init(void *states_dev, int64_t n, uint64_t seed, uint64_t subsequence_start,
                           const void *tables_dev, int64_t tables_bytes, void *stream) {
    B2K_RANGE("b2k_xoroshiro128p_init");
    if (n < 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_xoroshiro128p_init: negative n");
    if (n == 0) return B2K_OK;
    if (!states_dev) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_xoroshiro128p_init: null states");
    if (!b2k::aligned_to<void>(states_dev, 16))
        return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_xoroshiro128p_init: states must be 16-byte aligned");
    if (!tables_dev || tables_bytes < kTablesBytes || !b2k::aligned_to<void>(tables_dev, 16))
        return b2k::fail(B2K_ERR_SCRATCH, "b2k_xoroshiro128p_init: jump tables missing");
    const RingConstants &rc = ring();
    if (!rc.valid)
        return b2k::fail(B2K_ERR_UNSUPPORTED, "xoroshiro128p: jump recurrence self-check failed");

    // the 128 basis states of the seed (16 k generator steps): kept per thread for the
    // last seed, since shards and repeated initialisations reuse it
    thread_local bool basis_known = false;
    thread_local uint64_t basis_seed = 0;
    thread_local Basis basis;
    if (!basis_known || basis_seed != seed) {
        State u[128];
        basis_states(seed, u, 128);
        for (int j = 0; j < 128; ++j) {
            basis.w[j][0] = static_cast<uint32_t>(u[j].s0);
            basis.w[j][1] = static_cast<uint32_t>(u[j].s0 >> 32);
            basis.w[j][2] = static_cast<uint32_t>(u[j].s1);
            basis.w[j][3] = static_cast<uint32_t>(u[j].s1 >> 32);
        }
        basis_seed = seed;
        basis_known = true;
    }
    Poly4 p_low{{static_cast<uint32_t>(rc.p_low.lo), static_cast<uint32_t>(rc.p_low.lo >> 32),
                 static_cast<uint32_t>(rc.p_low.hi), static_cast<uint32_t>(rc.p_low.hi >> 32)}};

    if (n >= (int64_t(1) << 18) && B2K_ENV_INT("B2K_XORO_INIT_TABLES", 1) != 0) {
        static b2k::PerDeviceOnce once;   // the limit belongs to the device, not to the process
        const cudaError_t attr = once.run([] {
            return cudaFuncSetAttribute(xoro_init_table_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kTableBytes);
        });
        if (attr != cudaSuccess) return b2k::check_cuda(attr, "b2k_xoroshiro128p_init: smem attribute");
        // one contiguous run per thread over a grid that fills the GPU once; runs of
        // at least 64 states keep the y^index products a small share of the work
        const int64_t resident =
            static_cast<int64_t>(b2k::sm_count()) * B2K_ENV_INT("B2K_XORO_INIT_CTAS_PER_SM", 2) * 256;
        int64_t per_thread = (n + resident - 1) / resident;
        const int64_t floor_run = B2K_ENV_INT("B2K_XORO_INIT_PER_THREAD", 64);
        if (per_thread < floor_run) per_thread = floor_run;
        per_thread += per_thread & 1;
        if (per_thread > 0x7FFFFFFE) per_thread = 0x7FFFFFFE;
        const int64_t threads = (n + per_thread - 1) / per_thread;
        const int64_t grid = (threads + 255) / 256;
        if (grid > 0x7FFFFFFF) return b2k::fail(B2K_ERR_TOO_LARGE, "b2k_xoroshiro128p_init: too many states");
        const int wide = b2k::aligned_to<void>(states_dev, 32) ? 1 : 0;
        xoro_init_table_kernel<<<static_cast<unsigned>(grid), 256, kTableBytes, b2k::as_stream(stream)>>>(
            static_cast<uint4 *>(states_dev), n, subsequence_start, static_cast<int>(per_thread), wide,
            static_cast<const uint4 *>(tables_dev), basis, p_low);
    } else {
        // short arrays: runs of 16 amortise the table products, tiny ones stay parallel
        int per_thread = n >= (int64_t(1) << 16) ? 16 : 1;
        per_thread = B2K_ENV_INT("B2K_XORO_INIT_SHORT_PER_THREAD", per_thread);
        if (per_thread < 1) per_thread = 1;
        const int64_t threads = (n + per_thread - 1) / per_thread;
        const int64_t grid = (threads + 255) / 256;
        xoro_init_kernel<<<static_cast<unsigned>(grid), 256, 0, b2k::as_stream(stream)>>>(
            static_cast<uint4 *>(states_dev), n, subsequence_start, per_thread,
            static_cast<const uint4 *>(tables_dev), basis, p_low);
    }
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_xoroshiro128p_init launch");
    return B2K_OK;
}

int b2k_xoroshiro128p_fill(void *states_dev, int64_t n, int draw0, void *out0_dev, int64_t count0,
                           int draw1, void *out1_dev, int64_t count1, void *stream) {
    B2K_RANGE("b2k_xoroshiro128p_fill");
    if (n < 0 || count0 < 0 || count1 < 0)
        return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_xoroshiro128p_fill: negative size");
    if (n == 0 || (count0 == 0 && count1 == 0)) return B2K_OK;
    if (!states_dev || !b2k::aligned_to<void>(states_dev, 16))
        return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_xoroshiro128p_fill: states null or not 16-byte aligned");
    const int draws[2] = {draw0, draw1};
    void *outs[2] = {out0_dev, out1_dev};
    const int64_t counts[2] = {count0, count1};
    for (int k = 0; k < 2; ++k) {
        if (counts[k] == 0) continue;
        const size_t size = draw_size(draws[k]);
        if (size == 0) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_xoroshiro128p_fill: unknown draw %d", draws[k]);
        if (!outs[k]) return b2k::fail(B2K_ERR_INVALID_ARG, "b2k_xoroshiro128p_fill: null output");
        if (!b2k::aligned_to<void>(outs[k], size))
            return b2k::fail(B2K_ERR_ALIGNMENT, "b2k_xoroshiro128p_fill: output not aligned to its element size");
    }
    const int64_t groups = (n + 31) / 32;
    int64_t grid = (groups + kFillWarps - 1) / kFillWarps;
    const int64_t cap = static_cast<int64_t>(b2k::sm_count()) * B2K_ENV_INT("B2K_XORO_FILL_CTAS_PER_SM", 8);
    if (grid > cap) grid = cap;
    Segment a{out0_dev, count0, draw0}, b{out1_dev, count1, draw1};
    // four resident CTAs per SM at 64 registers; five or six (48 / 40 registers) measured
    // 2-5 % slower: the kernel is bound by the integer pipe and by issue slots, not by
    // latency that more warps could hide
    xoro_fill_kernel<4, 4><<<static_cast<unsigned>(grid), kFillWarps * 32, 0, b2k::as_stream(stream)>>>(
        static_cast<ulonglong2 *>(states_dev), n, a, b);
    b2k::note_launch();
    B2K_RETURN_IF_LAUNCH_FAILED("b2k_xoroshiro128p_fill launch");
    return B2K_OK;
}

}  // extern "C"
