// Drives the C++ host mirror (ascq_ascendc.hpp) end to end: reads operands from files, runs one operator on the
// GPU, writes the result to a file.  The Python test compares that file with the CPU oracle.
//   usage: ascendc_mirror_main <op> <dir>
//   op = quant_tensor | quant_channel | dequant_channel | antiquant_channel | quantize_token
#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "ascq_ascendc.hpp"

using namespace AscendC;

static std::vector<char> read_file(const std::string& path)
{
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}
static void write_file(const std::string& path, const void* p, size_t n)
{
    std::ofstream f(path, std::ios::binary);
    f.write(static_cast<const char*>(p), static_cast<std::streamsize>(n));
}
#define CU(x)                                                                          \
    do {                                                                               \
        cudaError_t e_ = (x);                                                          \
        if (e_ != cudaSuccess) throw std::runtime_error(std::string(#x) + ": " + cudaGetErrorString(e_)); \
    } while (0)

template <typename T> static GlobalTensor<T> upload(const std::vector<char>& h)
{
    void* d = nullptr;
    CU(cudaMalloc(&d, h.size() ? h.size() : 16));
    CU(cudaMemcpy(d, h.data(), h.size(), cudaMemcpyHostToDevice));
    return GlobalTensor<T>(static_cast<T*>(d), h.size() / sizeof(T));
}
template <typename T> static GlobalTensor<T> device_alloc(size_t n, int fill)
{
    void* d = nullptr;
    CU(cudaMalloc(&d, n * sizeof(T)));
    CU(cudaMemset(d, fill, n * sizeof(T)));
    return GlobalTensor<T>(static_cast<T*>(d), n);
}
template <typename T> static void download(const std::string& path, const GlobalTensor<T>& t)
{
    std::vector<char> h(t.size * sizeof(T));
    CU(cudaDeviceSynchronize());
    CU(cudaMemcpy(h.data(), t.ptr, h.size(), cudaMemcpyDeviceToHost));
    write_file(path, h.data(), h.size());
}

int main(int argc, char** argv)
{
    if (argc != 3) return 2;
    const std::string op = argv[1], dir = std::string(argv[2]) + "/";
    try {
        uint32_t dims[4] = {0, 0, 0, 0};
        if (op != "bad_args") {
            auto d = read_file(dir + "dims.bin");
            std::memcpy(dims, d.data(), d.size() < sizeof(dims) ? d.size() : sizeof(dims));
        }
        if (op == "quant_tensor") {  // dims: calCount; scale/offset in scalars.bin (2 floats)
            auto src = upload<half>(read_file(dir + "src.bin"));
            auto sc = read_file(dir + "scalars.bin");
            float s[2];
            std::memcpy(s, sc.data(), sizeof(s));
            auto dst = device_alloc<int8_t>(src.size, 0x55);
            AscendQuant<half>(dst, src, s[0], s[1], dims[0]);
            download(dir + "dst.bin", dst);
        } else if (op == "quant_channel") {  // dims: calCount, scaleCount
            auto src = upload<half>(read_file(dir + "src.bin"));
            auto scale = upload<half>(read_file(dir + "scale.bin"));
            auto offset = upload<half>(read_file(dir + "offset.bin"));
            auto dst = device_alloc<int8_t>(src.size, 0x55);
            AscendQuant<half>(dst, src, scale, offset, dims[1], dims[1], dims[0]);
            download(dir + "dst.bin", dst);
        } else if (op == "dequant_channel") {  // dims: m, n, calCount, dst row stride
            auto src = upload<int32_t>(read_file(dir + "src.bin"));
            auto scale = upload<float>(read_file(dir + "scale.bin"));
            auto dst = device_alloc<bfloat16_t>(size_t(dims[0]) * dims[3], 0);
            AscendDequant<bfloat16_t, float>(dst, src, scale, DequantParams{dims[0], dims[1], dims[2]});
            download(dir + "dst.bin", dst);
        } else if (op == "antiquant_channel") {  // dims: K, N
            auto src = upload<int8_t>(read_file(dir + "src.bin"));
            auto scale = upload<bfloat16_t>(read_file(dir + "scale.bin"));
            auto offset = upload<bfloat16_t>(read_file(dir + "offset.bin"));
            auto dst = device_alloc<bfloat16_t>(src.size, 0);
            AscendAntiQuant<int8_t, bfloat16_t, false>(dst, src, offset, scale, dims[0]);
            download(dir + "dst.bin", dst);
        } else if (op == "quantize_token") {  // dims: m, n; unified interface, PER_TOKEN with offset, float scales
            auto src = upload<half>(read_file(dir + "src.bin"));
            auto scale = upload<float>(read_file(dir + "scale.bin"));
            auto offset = upload<float>(read_file(dir + "offset.bin"));
            auto dst = device_alloc<int8_t>(src.size, 0x55);
            QuantizeConfig cfg{QuantizePolicy::PER_TOKEN, true, RoundMode::CAST_RINT, 1};
            Quantize(cfg, dst, src, scale, offset, QuantizeParams{dims[0], dims[1], 0});
            download(dir + "dst.bin", dst);
        } else if (op == "bad_args") {  // the reference asserts scaleCount == offsetCount
            GlobalTensor<int8_t> d;
            GlobalTensor<half> s;
            try {
                AscendQuant<half>(d, s, s, s, 8, 16, 64);
            } catch (const ascq::Error& e) {
                std::printf("status=%d\n", int(e.status));
                return e.status == ASCQ_ERR_INVALID_ARG ? 0 : 1;
            }
            return 1;
        } else {
            return 2;
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
