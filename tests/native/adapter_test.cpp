// Exercises the LiteNN-facing adapter the way LiteNN's own tests exercise the CUDA
// device (tests/CUDADeviceTest.cpp:108-125: compute on the device, compare with the
// CPU result).  Usage: adapter_test <fmt> <n> <k> <m> <payload.bin> <x.bin> <expected.bin>
// Runs dst = x . dequant(payload)^T through QuantizedMatMulCache::DoBinaryOp with device
// buffers, fp32 activations of any row count.  Prints "max_rel_err <value>" and exits 0,
// or "SKIP no CUDA device" with exit 77.
#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <vector>

#include "../../litenn_b200/host/LiteNNQuantMatMul.hpp"

using namespace LiteNN::B200;

template <typename T>
static std::vector<T> ReadAll(const char* path)
{
	std::ifstream f(path, std::ios::binary | std::ios::ate);
	if (!f)
	{
		throw std::runtime_error(std::string("cannot open ") + path);
	}
	const auto bytes = static_cast<std::size_t>(f.tellg());
	f.seekg(0);
	std::vector<T> out(bytes / sizeof(T));
	f.read(reinterpret_cast<char*>(out.data()), static_cast<std::streamsize>(bytes));
	return out;
}

int main(int argc, char** argv)
{
	// error behaviour first: it needs no GPU and must throw std::runtime_error
	try
	{
		std::vector<std::uint8_t> tiny(18);
		PackedWeight bad(CUDA{ 0 }, BlockQuantization(QuantizedBlockFormat::GGML_Q4_0, { 1, 48 }), tiny.data(), tiny.size());
		std::puts("FAIL: invalid row width accepted");
		return 1;
	}
	catch (const std::runtime_error& e)
	{
		if (std::string(e.what()).find("incompatible with ggml block size") == std::string::npos)
		{
			std::printf("FAIL: unexpected message: %s\n", e.what());
			return 1;
		}
	}
	if (qmm_device_count() == 0)
	{
		std::puts("SKIP no CUDA device");
		return 77;
	}
	if (argc != 8)
	{
		std::puts("usage: adapter_test fmt n k m payload x expected");
		return 2;
	}
	const auto fmt = static_cast<QuantizedBlockFormat>(std::atoi(argv[1]));
	const std::size_t n = std::strtoull(argv[2], nullptr, 10), k = std::strtoull(argv[3], nullptr, 10),
	                  m = std::strtoull(argv[4], nullptr, 10);
	const auto payload = ReadAll<std::uint8_t>(argv[5]);
	const auto x = ReadAll<float>(argv[6]);
	const auto expected = ReadAll<float>(argv[7]);

	CUDA device{ 0 };
	QuantizedMatMulCache cache;
	const auto params = BlockQuantization(fmt, { n, k });
	float *dx = nullptr, *dy = nullptr;
	if (cudaMalloc(reinterpret_cast<void**>(&dx), x.size() * sizeof(float)) != cudaSuccess ||
	    cudaMalloc(reinterpret_cast<void**>(&dy), m * n * sizeof(float)) != cudaSuccess ||
	    cudaMemcpy(dx, x.data(), x.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
	{
		std::puts("FAIL: device buffers");
		return 1;
	}
	std::vector<float> y(m * n);
	try
	{
		// the graph-level form: MatMul(activations, UInt8 payload described by QuantizationParams)
		cache.DoBinaryOp(device, BinaryOp::MatMul, dy, DataType::Float32, ShapeView{ m, k }, dx, DataType::UInt8,
		                 ShapeView{ payload.size() }, payload.data(), params);
		cache.DoBinaryOp(device, BinaryOp::MatMul, dy, DataType::Float32, ShapeView{ m, k }, dx, DataType::UInt8,
		                 ShapeView{ payload.size() }, payload.data(), params);
	}
	catch (const std::runtime_error& e)
	{
		std::printf("FAIL: %s\n", e.what());
		return 1;
	}
	if (cudaMemcpy(y.data(), dy, y.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess)
	{
		std::puts("FAIL: copy back");
		return 1;
	}
	// one packed weight for two runs on the same payload
	if (cache.Size() != 1)
	{
		std::puts("FAIL: the second run packed the weight again");
		return 1;
	}
	const PackedWeight first = cache.Get(device, params, payload.data(), payload.size());
	// the same address described as another tensor (half the rows) must not hit the first entry
	const auto half = BlockQuantization(fmt, { n / 2, k });
	const PackedWeight other = cache.Get(device, half, payload.data(), payload.size() / 2);
	if (other.Handle() == first.Handle() || cache.Size() != 2)
	{
		std::puts("FAIL: a reused address with another shape returned the stale weight");
		return 1;
	}
	if (cache.Invalidate(payload.data()) != 2 || cache.Size() != 0)
	{
		std::puts("FAIL: Invalidate did not drop the payload's entries");
		return 1;
	}
	// wrong inner dimension: the MatMul shape rule (src/LiteNN/Operators.h:197-222)
	try
	{
		cache.DoBinaryOp(device, BinaryOp::MatMul, dy, DataType::Float32, ShapeView{ m, k + 32 }, dx, DataType::UInt8,
		                 ShapeView{ payload.size() }, payload.data(), params);
		std::puts("FAIL: mismatched inner dimension accepted");
		return 1;
	}
	catch (const std::runtime_error&)
	{
	}
	cudaFree(dx);
	cudaFree(dy);
	double max_e = 0, max_abs = 0;
	for (std::size_t i = 0; i < y.size(); ++i)
	{
		max_e = std::max(max_e, std::fabs(static_cast<double>(y[i]) - expected[i]));
		max_abs = std::max(max_abs, std::fabs(static_cast<double>(expected[i])));
	}
	std::printf("max_rel_err %.3e\n", max_abs > 0 ? max_e / max_abs : max_e);
	return 0;
}
