// Stand-alone C++ driver on the C++ host mirror (include/kleos_b200.hpp), written the way the
// reference's own driver is (csrc/main.cu:12-73 runOS): initialise, build the packed input
// buffer [A | Wg | W1 | W2 | b1 | b2] in fp32 on the host, convert it to the layer's element
// type, copy it to the device, time the forward with forwardHostBench<32, 32>, print
// "epRank: <rank> took <ms>ms", finalise.
//
//   kleos_driver                       timed run on random inputs (the reference's only mode)
//   kleos_driver --io IN.bin OUT.bin   one forward on the packed input image in IN.bin (already
//                                      in the element type), packed output image to OUT.bin;
//                                      used by the parity test
// The layer comes from kleos_config.json in the working directory or from $KLEOS_CONFIG; rank
// and world size from the launcher's environment.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <fstream>
#include <random>
#include <vector>

#include "../../include/kleos_b200.hpp"

#define DRIVER_CHECK_CUDA(e)                                                                 \
    do {                                                                                     \
        cudaError_t code = (e);                                                              \
        if (code != cudaSuccess) {                                                           \
            std::fprintf(stderr, "<%s:%d> %s: %s\n", __FILE__, __LINE__, #e, cudaGetErrorString(code)); \
            std::exit(1);                                                                    \
        }                                                                                    \
    } while (0)

namespace {

// fp32 -> the layer's element type, into a byte image (the reference converts in place with
// cutlass::NumericConverter, main.cu:58-61)
std::vector<unsigned char> convert(const std::vector<float>& src, int torch_dtype) {
    const size_t n = src.size();
    std::vector<unsigned char> out(n * ((torch_dtype == 0 || torch_dtype == 1) ? 4 : 2));
    if (torch_dtype == 0) {
        std::memcpy(out.data(), src.data(), n * 4);
    } else if (torch_dtype == 1) {  // TF32: 10-bit mantissa, round to nearest even
        auto* o = reinterpret_cast<uint32_t*>(out.data());
        for (size_t i = 0; i < n; ++i) {
            uint32_t u;
            std::memcpy(&u, &src[i], 4);
            if ((u & 0x7f800000u) != 0x7f800000u) u = (u + 0xfffu + ((u >> 13) & 1u)) & 0xffffe000u;
            o[i] = u;
        }
    } else if (torch_dtype == 2) {
        auto* o = reinterpret_cast<__nv_bfloat16*>(out.data());
        for (size_t i = 0; i < n; ++i) o[i] = __float2bfloat16_rn(src[i]);
    } else {
        auto* o = reinterpret_cast<__half*>(out.data());
        for (size_t i = 0; i < n; ++i) o[i] = __float2half_rn(src[i]);
    }
    return out;
}

std::vector<unsigned char> read_file(const char* path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) {
        std::fprintf(stderr, "cannot open %s\n", path);
        std::exit(1);
    }
    std::vector<unsigned char> v(static_cast<size_t>(f.tellg()));
    f.seekg(0);
    f.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(v.size()));
    return v;
}

}  // namespace

int main(int argc, char** argv) {
    const bool io = argc == 4 && std::strcmp(argv[1], "--io") == 0;
    if (argc != 1 && !io) {
        std::fprintf(stderr, "usage: %s [--io IN.bin OUT.bin]\n", argv[0]);
        return 2;
    }
    kleos::initialize();
    const auto rank = kleos::getRank();
    const kleos_layer_info L = kleos::layerInfo();
    const size_t eb = static_cast<size_t>(L.elem_bytes);
    const size_t in_bytes = static_cast<size_t>(L.input_elems) * eb, out_bytes = static_cast<size_t>(L.output_elems) * eb;

    std::vector<unsigned char> image;
    if (io) {
        image = read_file(argv[2]);
        if (image.size() != in_bytes) {
            std::fprintf(stderr, "%s holds %zu bytes, the layer's packed input is %zu\n", argv[2], image.size(), in_bytes);
            return 1;
        }
    } else {
        // activations, gate and expert weights from N(0, 1/sqrt(fan_in))-like draws, zero biases;
        // the seed depends on the rank as in the reference (main.cu:42)
        std::vector<float> host(static_cast<size_t>(L.input_elems), 0.f);
        std::mt19937 rng(47u * (rank + 42u));
        std::normal_distribution<float> dist(0.f, 1.f);
        const size_t a_end = static_cast<size_t>(L.S) * L.H;
        const bool dense = L.E == 1;
        const size_t wg_end = a_end + (dense ? 0 : static_cast<size_t>(L.E) * L.H);
        const size_t w_begin = a_end + (dense ? 0 : static_cast<size_t>(L.PX) * L.H);
        const size_t w_end = w_begin + 2 * static_cast<size_t>(L.local_experts) * L.I * L.H;
        for (size_t i = 0; i < a_end; ++i) host[i] = dist(rng);
        for (size_t i = a_end; i < wg_end; ++i) host[i] = dist(rng) * 0.02f;
        for (size_t i = w_begin; i < w_end; ++i) host[i] = dist(rng) * 0.02f;
        image = convert(host, L.torch_dtype);
    }

    unsigned char *iP = nullptr, *oP = nullptr;
    DRIVER_CHECK_CUDA(cudaMalloc(&iP, in_bytes));
    DRIVER_CHECK_CUDA(cudaMalloc(&oP, out_bytes));
    DRIVER_CHECK_CUDA(cudaMemset(oP, 0, out_bytes));
    DRIVER_CHECK_CUDA(cudaMemcpy(iP, image.data(), in_bytes, cudaMemcpyHostToDevice));

    if (io) {
        kleos::moe::forwardHost(iP, oP);
        DRIVER_CHECK_CUDA(cudaStreamSynchronize(cudaStreamPerThread));
        kleos_status st{};
        if (kleos_last_status(&st) != KLEOS_OK || st.code != 0) {
            std::fprintf(stderr, "device status: code=%d where=%d detail=%d\n", st.code, st.where, st.detail);
            return 1;
        }
        std::vector<unsigned char> result(out_bytes);
        DRIVER_CHECK_CUDA(cudaMemcpy(result.data(), oP, out_bytes, cudaMemcpyDeviceToHost));
        std::ofstream f(argv[3], std::ios::binary | std::ios::trunc);
        f.write(reinterpret_cast<const char*>(result.data()), static_cast<std::streamsize>(result.size()));
    } else {
        float timed = 0;
        kleos::moe::forwardHostBench<32, 32>(iP, oP, timed);
        std::printf("epRank: %u took %.2fms\n", rank, timed);
    }
    DRIVER_CHECK_CUDA(cudaPeekAtLastError());
    DRIVER_CHECK_CUDA(cudaFree(iP));
    DRIVER_CHECK_CUDA(cudaFree(oP));
    kleos::finalize();
    return 0;
}
