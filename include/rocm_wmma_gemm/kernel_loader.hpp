// Run-time loader of the GEMM shared object.  Same class, constructor behaviour and `gemm`
// member templates as the reference's rocm_wmma_gemm::loader
// (rocm_wmma_gemm/include/rocm_wmma_gemm/kernel_loader.hpp:28-186): it asks device 0 for its
// architecture, dlopen()s `librocm_wmma_gemm_<arch>.so` (first from ROCM_WMMA_GEMM_LIB_DIR if
// that macro is defined, then from the dynamic linker's search path), resolves the four
// `rocm_wmma_gemm_<out>_<in>` C symbols and dispatches through them.  On CUDA the
// architecture string is "sm" + compute capability + "a" for the arch-specific build, i.e.
// "sm100a" on B200.  Header-only; link with -ldl -lcudart.
#ifndef ROCM_WMMA_GEMM_KERNEL_LOADER_HPP
#define ROCM_WMMA_GEMM_KERNEL_LOADER_HPP

#include <dlfcn.h>
#include <rocm_wmma_gemm/kernel/common.hpp>
#include <stdexcept>
#include <string>
#include <type_traits>

namespace rocm_wmma_gemm
{

class loader
{
    using dispatch_fn = void (*)(void*, void*, void*, size_t, size_t, size_t, size_t, int, int, int, void*);
    using status_fn   = int (*)();
    using message_fn  = const char* (*)();

    void*       handle_     = nullptr;
    dispatch_fn dispatch_[4] = {nullptr, nullptr, nullptr, nullptr};
    status_fn   last_status_ = nullptr;
    message_fn  last_error_  = nullptr;

    template<class F>
    static F resolve(void* handle, const char* name, bool required = true)
    {
        auto fn = reinterpret_cast<F>(dlsym(handle, name));
        if(!fn && required)
            throw std::runtime_error(std::string("rocm_wmma_gemm::loader: symbol not found: ") + name);
        return fn;
    }

public:
    loader()
    {
        cudaDeviceProp props{};
        if(cudaGetDeviceProperties(&props, 0) != cudaSuccess)
            throw std::runtime_error("rocm_wmma_gemm::loader: cudaGetDeviceProperties failed");
        const std::string arch    = "sm" + std::to_string(props.major * 10 + props.minor) + "a";
        const std::string libname = "librocm_wmma_gemm_" + arch + ".so";
#ifdef ROCM_WMMA_GEMM_LIB_DIR
        handle_ = dlopen((std::string(ROCM_WMMA_GEMM_LIB_DIR "/") + libname).c_str(), RTLD_NOW | RTLD_LOCAL);
#endif
        if(!handle_) handle_ = dlopen(libname.c_str(), RTLD_NOW | RTLD_LOCAL);
        if(!handle_)
        {
            const char* why = dlerror();
            throw std::runtime_error("rocm_wmma_gemm::loader: could not open " + libname + ": " + (why ? why : "?"));
        }
        dispatch_[0] = resolve<dispatch_fn>(handle_, "rocm_wmma_gemm_f16_f16");
        dispatch_[1] = resolve<dispatch_fn>(handle_, "rocm_wmma_gemm_f32_f16");
        dispatch_[2] = resolve<dispatch_fn>(handle_, "rocm_wmma_gemm_bf16_bf16");
        dispatch_[3] = resolve<dispatch_fn>(handle_, "rocm_wmma_gemm_f32_bf16");
        // Optional: lets callers see why a (void) reference entry point did nothing.
        last_status_ = resolve<status_fn>(handle_, "b200_gemm_last_status", false);
        last_error_  = resolve<message_fn>(handle_, "b200_gemm_last_error", false);
    }

    ~loader()
    {
        if(handle_) dlclose(handle_);
    }

    loader(const loader&)            = delete;
    loader& operator=(const loader&) = delete;
    loader(loader&&)                 = delete;
    loader& operator=(loader&&)      = delete;

    template<m_layout layout_C, m_layout layout_A, m_layout layout_B, class T, class U>
    void gemm(T* C, U* A, U* B, size_t M, size_t N, size_t K, hipStream_t& stream)
    {
        gemm<layout_C, layout_A, layout_B>(C, A, B, M, N, K, 1, stream);
    }

    template<m_layout layout_C, m_layout layout_A, m_layout layout_B, class T, class U>
    void gemm(T* C, U* A, U* B, size_t M, size_t N, size_t K, size_t batch_count, hipStream_t& stream)
    {
        select_fn<T, U>()(C,
                          A,
                          B,
                          M,
                          N,
                          K,
                          batch_count,
                          layout_C == m_layout::col_major ? 1 : 0,
                          layout_A == m_layout::col_major ? 1 : 0,
                          layout_B == m_layout::col_major ? 1 : 0,
                          &stream);
    }

    // Status (0 = ok) and message of the calling thread's last failing call; not in the
    // reference, whose entry points have no way to report a failure.
    int last_status() const
    {
        return last_status_ ? last_status_() : 0;
    }
    const char* last_error() const
    {
        return last_error_ ? last_error_() : "";
    }

private:
    template<class T, class U>
    dispatch_fn select_fn() const
    {
        if constexpr(std::is_same_v<T, half> && std::is_same_v<U, half>) return dispatch_[0];
        else if constexpr(std::is_same_v<T, float> && std::is_same_v<U, half>) return dispatch_[1];
        else if constexpr(std::is_same_v<T, __hip_bfloat16> && std::is_same_v<U, __hip_bfloat16>)
            return dispatch_[2];
        else if constexpr(std::is_same_v<T, float> && std::is_same_v<U, __hip_bfloat16>) return dispatch_[3];
        else
        {
            static_assert(sizeof(T) == 0, "Unsupported type pair for rocm_wmma_gemm::loader");
            return nullptr;
        }
    }
};

} // namespace rocm_wmma_gemm

#endif // ROCM_WMMA_GEMM_KERNEL_LOADER_HPP
