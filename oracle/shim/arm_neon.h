/* Empty stand-in so that the reference's src/matmul_simd.cpp, which includes
 * <arm_neon.h> above its __aarch64__ guard, preprocesses on an x86 host.
 * The guarded NEON code is never compiled here. */
