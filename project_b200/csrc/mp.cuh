// 32-bit multi-precision primitives for sm_100a.
//
// Every big-number routine in this library is written on top of the carry-flag
// instructions below (add.cc / addc / mad.lo.cc / madc.hi.cc ...), which map to
// the integer multiply-add pipe with hardware carry.  When the header is
// compiled for the host (unit tests of the carry-chain logic, no GPU needed) the
// same routines run on an emulated carry flag.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define GZK_HD __host__ __device__ __forceinline__
#define GZK_D __device__ __forceinline__
#else
#define GZK_HD inline
#define GZK_D inline
#endif

namespace gzk
{
    namespace mp
    {
#if defined(__CUDA_ARCH__)
        GZK_D uint32_t add_cc(uint32_t a, uint32_t b)
        {
            uint32_t r;
            asm volatile("add.cc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint32_t addc_cc(uint32_t a, uint32_t b)
        {
            uint32_t r;
            asm volatile("addc.cc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint32_t addc(uint32_t a, uint32_t b)
        {
            uint32_t r;
            asm volatile("addc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint32_t sub_cc(uint32_t a, uint32_t b)
        {
            uint32_t r;
            asm volatile("sub.cc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint32_t subc_cc(uint32_t a, uint32_t b)
        {
            uint32_t r;
            asm volatile("subc.cc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint32_t subc(uint32_t a, uint32_t b)
        {
            uint32_t r;
            asm volatile("subc.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint32_t mul_lo(uint32_t a, uint32_t b)
        {
            uint32_t r;
            asm volatile("mul.lo.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint32_t mul_hi(uint32_t a, uint32_t b)
        {
            uint32_t r;
            asm volatile("mul.hi.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint32_t mad_lo_cc(uint32_t a, uint32_t b, uint32_t c)
        {
            uint32_t r;
            asm volatile("mad.lo.cc.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
            return r;
        }
        GZK_D uint32_t mad_hi_cc(uint32_t a, uint32_t b, uint32_t c)
        {
            uint32_t r;
            asm volatile("mad.hi.cc.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
            return r;
        }
        GZK_D uint32_t madc_lo_cc(uint32_t a, uint32_t b, uint32_t c)
        {
            uint32_t r;
            asm volatile("madc.lo.cc.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
            return r;
        }
        GZK_D uint32_t madc_hi_cc(uint32_t a, uint32_t b, uint32_t c)
        {
            uint32_t r;
            asm volatile("madc.hi.cc.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
            return r;
        }
        GZK_D uint32_t madc_hi(uint32_t a, uint32_t b, uint32_t c)
        {
            uint32_t r;
            asm volatile("madc.hi.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
            return r;
        }
        GZK_D uint64_t mul_wide(uint32_t a, uint32_t b)
        {
            uint64_t r;
            asm volatile("mul.wide.u32 %0, %1, %2;" : "=l"(r) : "r"(a), "r"(b));
            return r;
        }
        GZK_D uint64_t add_cc_u64(uint64_t a, uint64_t b)
        {
            uint64_t r;
            asm volatile("add.cc.u64 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
            return r;
        }
        GZK_D uint64_t addc_cc_u64(uint64_t a, uint64_t b)
        {
            uint64_t r;
            asm volatile("addc.cc.u64 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
            return r;
        }
#else
        // Host emulation of the carry flag (single-threaded use per thread).
        inline uint32_t& cc_flag()
        {
            static thread_local uint32_t flag = 0;
            return flag;
        }
        inline uint32_t emu_add(uint32_t a, uint32_t b, uint32_t cin, bool set)
        {
            const uint64_t t = static_cast<uint64_t>(a) + b + cin;
            if (set) cc_flag() = static_cast<uint32_t>(t >> 32);
            return static_cast<uint32_t>(t);
        }
        inline uint32_t emu_sub(uint32_t a, uint32_t b, uint32_t bin, bool set)
        {
            const uint64_t t = static_cast<uint64_t>(a) - b - bin;
            // PTX sub.cc leaves the *borrow* in CC.CF; subc consumes it as a borrow.
            if (set) cc_flag() = static_cast<uint32_t>((t >> 32) & 1U);
            return static_cast<uint32_t>(t);
        }
        inline uint32_t add_cc(uint32_t a, uint32_t b) { return emu_add(a, b, 0, true); }
        inline uint32_t addc_cc(uint32_t a, uint32_t b) { return emu_add(a, b, cc_flag(), true); }
        inline uint32_t addc(uint32_t a, uint32_t b) { return emu_add(a, b, cc_flag(), false); }
        inline uint32_t sub_cc(uint32_t a, uint32_t b) { return emu_sub(a, b, 0, true); }
        inline uint32_t subc_cc(uint32_t a, uint32_t b) { return emu_sub(a, b, cc_flag(), true); }
        inline uint32_t subc(uint32_t a, uint32_t b) { return emu_sub(a, b, cc_flag(), false); }
        inline uint32_t mul_lo(uint32_t a, uint32_t b) { return static_cast<uint32_t>(static_cast<uint64_t>(a) * b); }
        inline uint32_t mul_hi(uint32_t a, uint32_t b) { return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32); }
        inline uint32_t mad_lo_cc(uint32_t a, uint32_t b, uint32_t c) { return emu_add(mul_lo(a, b), c, 0, true); }
        inline uint32_t mad_hi_cc(uint32_t a, uint32_t b, uint32_t c) { return emu_add(mul_hi(a, b), c, 0, true); }
        inline uint32_t madc_lo_cc(uint32_t a, uint32_t b, uint32_t c) { return emu_add(mul_lo(a, b), c, cc_flag(), true); }
        inline uint32_t madc_hi_cc(uint32_t a, uint32_t b, uint32_t c) { return emu_add(mul_hi(a, b), c, cc_flag(), true); }
        inline uint32_t madc_hi(uint32_t a, uint32_t b, uint32_t c) { return emu_add(mul_hi(a, b), c, cc_flag(), false); }
        inline uint64_t mul_wide(uint32_t a, uint32_t b) { return static_cast<uint64_t>(a) * b; }
        inline uint64_t emu_add64(uint64_t a, uint64_t b, uint32_t cin)
        {
            const unsigned __int128 t = static_cast<unsigned __int128>(a) + b + cin;
            cc_flag() = static_cast<uint32_t>(t >> 64);
            return static_cast<uint64_t>(t);
        }
        inline uint64_t add_cc_u64(uint64_t a, uint64_t b) { return emu_add64(a, b, 0); }
        inline uint64_t addc_cc_u64(uint64_t a, uint64_t b) { return emu_add64(a, b, cc_flag()); }
#endif
    }
}
