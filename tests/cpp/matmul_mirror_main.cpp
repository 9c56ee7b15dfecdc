// Drives the C++ host mirror of the Matmul object (ascq_matmul.hpp) end to end, written the way the reference's
// samples use the object (matmul_quant.asc:105-135, matmul_mx.asc): reads operands from files, runs one matmul on
// the GPU, writes C to a file.  The Python test compares that file with the CPU oracle.
//   usage: matmul_mirror_main <case> <dir>        dims.bin holds M, N, K as uint32
#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "ascq_matmul.hpp"

using namespace AscendC;

static std::vector<char> read_file(const std::string& path)
{
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}
#define CU(x)                                                                          \
    do {                                                                               \
        cudaError_t e_ = (x);                                                          \
        if (e_ != cudaSuccess) throw std::runtime_error(std::string(#x) + ": " + cudaGetErrorString(e_)); \
    } while (0)

template <typename T> static GlobalTensor<T> upload(const std::string& path)
{
    const std::vector<char> h = read_file(path);
    void* d = nullptr;
    CU(cudaMalloc(&d, h.size() ? h.size() : 16));
    CU(cudaMemcpy(d, h.data(), h.size(), cudaMemcpyHostToDevice));
    return GlobalTensor<T>(static_cast<T*>(d), h.size() / sizeof(T));
}
template <typename T> static GlobalTensor<T> device_alloc(size_t n)
{
    void* d = nullptr;
    CU(cudaMalloc(&d, n * sizeof(T) + 16));
    CU(cudaMemset(d, 0x5A, n * sizeof(T)));
    return GlobalTensor<T>(static_cast<T*>(d), n);
}
template <typename T> static void download(const std::string& path, const GlobalTensor<T>& t)
{
    std::vector<char> h(t.size * sizeof(T));
    CU(cudaDeviceSynchronize());
    ascq::check(ascq_matmul_status(nullptr));
    CU(cudaMemcpy(h.data(), t.ptr, h.size(), cudaMemcpyDeviceToHost));
    std::ofstream f(path, std::ios::binary);
    f.write(h.data(), static_cast<std::streamsize>(h.size()));
}

template <typename T, bool TRANS = false> using Gm = MatmulType<TPosition::GM, CubeFormat::ND, T, TRANS>;
template <typename T, bool TRANS = false> using GmMx = MatmulTypeWithScale<TPosition::GM, TPosition::GM, CubeFormat::ND, T, TRANS>;

int main(int argc, char** argv)
{
    if (argc != 3) return 2;
    const std::string op = argv[1], dir = std::string(argv[2]) + "/";
    try {
        uint32_t d[3] = {0, 0, 0};
        if (op != "errors") {
            const auto raw = read_file(dir + "dims.bin");
            std::memcpy(d, raw.data(), sizeof(d));
        }
        const int M = int(d[0]), N = int(d[1]), K = int(d[2]);
        TCubeTiling tiling;
        tiling.M = M; tiling.N = N; tiling.Ka = K; tiling.Kb = K;
        tiling.singleCoreM = M; tiling.singleCoreN = N; tiling.singleCoreK = K;

        if (op == "quant_vector" || op == "quant_scalar") {
            // matmul_quant sample: int8 x int8 -> half, int32 bias, B stored [K, N]; quantisation per channel or 0.1
            Matmul<Gm<int8_t>, Gm<int8_t>, Gm<half>, Gm<int32_t>> mm;
            tiling.isBias = 1;
            mm.Init(&tiling);
            auto a = upload<int8_t>(dir + "a.bin"), b = upload<int8_t>(dir + "b_kn.bin");
            auto bias = upload<int32_t>(dir + "bias.bin");
            auto c = device_alloc<half>(size_t(M) * N);
            auto ws = device_alloc<uint8_t>(mm.GetWorkspaceSize());
            mm.SetWorkspace(ws);
            mm.SetTensorA(a);
            mm.SetTensorB(b);
            mm.SetBias(bias);
            if (op == "quant_vector") {
                mm.SetQuantVector(upload<uint64_t>(dir + "quant.bin"));
            } else {
                float quantFloat = 0.1f;
                uint32_t bits;
                std::memcpy(&bits, &quantFloat, 4);
                mm.SetQuantScalar(static_cast<uint64_t>(bits));
            }
            mm.IterateAll(c);
            mm.End();
            download(dir + "c.bin", c);
        } else if (op == "requant_vector") {
            // int8 x int8 -> int8, B K-major, the Iterate / GetTensorC form
            Matmul<Gm<int8_t>, Gm<int8_t, true>, Gm<int8_t>, Gm<int32_t>> mm;
            mm.SetOrgShape(M, N, K);
            auto a = upload<int8_t>(dir + "a.bin"), b = upload<int8_t>(dir + "b_nk.bin");
            auto c = device_alloc<int8_t>(size_t(M) * N);
            mm.SetTensorA(a);
            mm.SetTensorB(b, true);
            mm.SetQuantVector(upload<uint64_t>(dir + "quant.bin"));
            int blocks = 0;
            while (mm.Iterate()) {
                mm.GetTensorC(c);
                ++blocks;
            }
            mm.End();
            if (blocks != 1) throw std::runtime_error("expected one iteration");
            download(dir + "c.bin", c);
        } else if (op == "f16_quant") {
            // half x half -> int8 through the quantising output (fixpipe sample, fp32 accumulator), B stored [K, N] is 16-bit:
            // the test hands it over K-major
            Matmul<Gm<half>, Gm<half, true>, Gm<int8_t>> mm;
            mm.Init(&tiling);
            auto a = upload<half>(dir + "a.bin"), b = upload<half>(dir + "b_nk.bin");
            auto c = device_alloc<int8_t>(size_t(M) * N);
            mm.SetTensorA(a);
            mm.SetTensorB(b, true);
            mm.SetQuantVector(upload<uint64_t>(dir + "quant.bin"));
            mm.IterateAll(c);
            download(dir + "c.bin", c);
        } else if (op == "acc_i32") {
            Matmul<Gm<int8_t>, Gm<int8_t, true>, Gm<int32_t>, Gm<int32_t>> mm;
            mm.Init(&tiling);
            auto a = upload<int8_t>(dir + "a.bin"), b = upload<int8_t>(dir + "b_nk.bin");
            auto c = device_alloc<int32_t>(size_t(M) * N);
            mm.SetTensorA(a);
            mm.SetTensorB(b, true);
            mm.IterateAll(c);
            download(dir + "c.bin", c);
        } else if (op == "bf16") {
            Matmul<Gm<bfloat16_t>, Gm<bfloat16_t, true>, Gm<float>> mm;
            mm.Init(&tiling);
            auto a = upload<bfloat16_t>(dir + "a.bin"), b = upload<bfloat16_t>(dir + "b_nk.bin");
            auto c = device_alloc<float>(size_t(M) * N);
            mm.SetTensorA(a);
            mm.SetTensorB(b, true);
            mm.IterateAll(c);
            download(dir + "c.bin", c);
        } else if (op == "w8a16") {
            // half x int8 with per-channel antiquant vectors, weight stored [K, N]
            Matmul<Gm<half>, Gm<int8_t>, Gm<half>> mm;
            mm.Init(&tiling);
            auto a = upload<half>(dir + "a.bin");
            auto b = upload<int8_t>(dir + "b_kn.bin");
            auto c = device_alloc<half>(size_t(M) * N);
            mm.SetTensorA(a);
            mm.SetTensorB(b);
            mm.SetAntiQuantVector(upload<half>(dir + "offset.bin"), upload<half>(dir + "scale.bin"));
            auto ws = device_alloc<uint8_t>(mm.GetWorkspaceSize());
            mm.SetWorkspace(ws);
            mm.IterateAll(c);
            download(dir + "c.bin", c);
        } else if (op == "mxfp4") {
            // matmul_mxfp4 sample's layouts: B [K, N] fp4 pairs along N, scaleB [K/64, N, 2]
            Matmul<GmMx<fp4x2_e2m1_t>, GmMx<fp4x2_e2m1_t>, Gm<bfloat16_t>> mm;
            mm.Init(&tiling);
            auto a = upload<fp4x2_e2m1_t>(dir + "a.bin"), b = upload<fp4x2_e2m1_t>(dir + "b_kn.bin");
            auto c = device_alloc<bfloat16_t>(size_t(M) * N);
            mm.SetTensorA(a);
            mm.SetTensorB(b);
            mm.SetTensorScaleA(upload<fp8_e8m0_t>(dir + "sa.bin"));
            mm.SetTensorScaleB(upload<fp8_e8m0_t>(dir + "sb_ref.bin"), false);
            auto ws = device_alloc<uint8_t>(mm.GetWorkspaceSize());
            mm.SetWorkspace(ws);
            mm.IterateAll(c);
            download(dir + "c.bin", c);
        } else if (op == "mxfp8") {
            Matmul<GmMx<fp8_e4m3fn_t>, GmMx<fp8_e5m2_t, true>, Gm<float>> mm;
            mm.Init(&tiling);
            auto a = upload<fp8_e4m3fn_t>(dir + "a.bin");
            auto b = upload<fp8_e5m2_t>(dir + "b_nk.bin");
            auto c = device_alloc<float>(size_t(M) * N);
            mm.SetTensorA(a);
            mm.SetTensorB(b, true);
            mm.SetTensorScaleA(upload<fp8_e8m0_t>(dir + "sa.bin"));
            mm.SetTensorScaleB(upload<fp8_e8m0_t>(dir + "sb.bin"));
            auto ws = device_alloc<uint8_t>(mm.GetWorkspaceSize());
            mm.SetWorkspace(ws);
            mm.IterateAll(c);
            download(dir + "c.bin", c);
        } else if (op == "errors") {
            // what the reference asserts comes back as ascq::Error; no GPU is touched
            int caught = 0;
            GlobalTensor<int8_t> a8(reinterpret_cast<int8_t*>(0x1000), 64), c8(reinterpret_cast<int8_t*>(0x3000), 64);
            {
                Matmul<Gm<int8_t>, Gm<int8_t, true>, Gm<int8_t>, Gm<int32_t>> mm;  // quantised output without quant parameters
                mm.SetOrgShape(8, 8, 16);
                mm.SetTensorA(a8);
                mm.SetTensorB(a8, true);
                try { mm.IterateAll(c8); } catch (const ascq::Error& e) { caught += e.status == ASCQ_ERR_INVALID_ARG; }
            }
            {
                Matmul<Gm<half>, Gm<half>, Gm<half>> mm;  // 16-bit B in [K, N] form
                GlobalTensor<half> h(reinterpret_cast<half*>(0x1000), 64);
                mm.SetOrgShape(8, 8, 16);
                mm.SetTensorA(h);
                mm.SetTensorB(h);
                try { mm.IterateAll(h); } catch (const ascq::Error& e) { caught += e.status == ASCQ_ERR_UNSUPPORTED; }
            }
            {
                Matmul<Gm<int8_t>, Gm<int8_t, true>, Gm<int32_t>, Gm<int32_t>> mm;  // GetTensorC with no block pending
                GlobalTensor<int32_t> c(reinterpret_cast<int32_t*>(0x1000), 64);
                try { mm.GetTensorC(c); } catch (const ascq::Error& e) { caught += e.status == ASCQ_ERR_INVALID_ARG; }
            }
            std::printf("caught=%d\n", caught);
            return caught == 3 ? 0 : 1;
        } else {
            return 2;
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
