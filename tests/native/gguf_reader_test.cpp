// Drives the ggml-free GGUF reader (litenn_b200/host/GGUFReader.hpp) the way the reference's
// importer test drives ImportGGUFArchive (tests/GGUFImporterTest.cpp:469-535): open an archive,
// list metadata and tensors, read payloads.
//   gguf_reader_test list <file>                      one line per metadata entry and tensor
//   gguf_reader_test payload <file> <tensor> <out>    the tensor's stored bytes -> <out>
//   gguf_reader_test pack <file> <tensor> <out>       file -> upload-time repack on GPU 0 -> dequantized fp32 -> <out>
//                                                     (exit 77 without a CUDA device)
//   gguf_reader_test dequant <file> <tensor> <out>    file -> raw payload on GPU 0 -> dequantized fp32 -> <out>
//                                                     (any known block format, also those without matmul kernels)
// A std::runtime_error is printed as "ERROR <message>" with exit code 3.
#include <cuda_runtime_api.h>

#include <cstdio>
#include <fstream>
#include <iostream>
#include <string>

#include "../../litenn_b200/host/GGUFReader.hpp"

using namespace LiteNN::B200;

static void PrintValue(const GGUF::MetadataValue& v)
{
	std::visit(
	    [](const auto& x) {
		    using T = std::decay_t<decltype(x)>;
		    if constexpr (std::is_same_v<T, std::string>)
		    {
			    std::cout << "str " << x;
		    }
		    else if constexpr (std::is_same_v<T, bool>)
		    {
			    std::cout << "bool " << (x ? 1 : 0);
		    }
		    else if constexpr (std::is_same_v<T, std::uint64_t>)
		    {
			    std::cout << "u64 " << x;
		    }
		    else if constexpr (std::is_same_v<T, std::int64_t>)
		    {
			    std::cout << "i64 " << x;
		    }
		    else if constexpr (std::is_same_v<T, double>)
		    {
			    std::cout << "f64 " << x;
		    }
		    else
		    {
			    std::cout << "array " << x.size();
			    for (const auto& e : x)
			    {
				    std::cout << " " << e;
			    }
		    }
	    },
	    v);
}

int main(int argc, char** argv)
{
	try
	{
		if (argc < 3)
		{
			std::puts("usage: gguf_reader_test list|payload|pack <file> [tensor out]");
			return 2;
		}
		const std::string mode = argv[1];
		GGUF::Archive archive(argv[2]);
		if (mode == "list")
		{
			std::cout << "version " << archive.Version() << "\n";
			for (const auto& e : archive.Metadata())
			{
				std::cout << "meta " << e.key << " ";
				PrintValue(e.value);
				std::cout << "\n";
			}
			for (const auto& t : archive.Tensors())
			{
				std::cout << "tensor " << t.name << " type " << static_cast<std::uint32_t>(t.type) << " format "
				          << (t.blockFormat ? static_cast<int>(*t.blockFormat) : -1) << " bytes " << t.bytes << " shape";
				for (const auto d : t.shape)
				{
					std::cout << " " << d;
				}
				const auto payload = archive.ReadPayload(t);
				std::cout << " first " << static_cast<int>(payload.front()) << " last " << static_cast<int>(payload.back())
				          << "\n";
			}
			const auto h = archive.ParseLLaMAHyperparameters();
			std::cout << "hparams " << h.architecture << " " << h.contextLength << " " << h.embeddingLength << " "
			          << h.blockCount << " " << h.feedForwardLength << " " << h.attentionHeadCount << " "
			          << h.attentionHeadCountKV << " " << h.HeadDimension() << " " << h.QueryGroupsPerKVHead() << " "
			          << h.ropeDimensionCount << " " << h.ropeFrequencyBase << " " << h.rmsNormEpsilon << "\n";
			return 0;
		}
		if (argc != 5)
		{
			std::puts("usage: gguf_reader_test payload|pack|dequant <file> <tensor> <out>");
			return 2;
		}
		const auto& t = archive.Tensor(argv[3]);
		std::ofstream out(argv[4], std::ios::binary);
		if (mode == "payload")
		{
			const auto payload = archive.ReadPayload(t);
			out.write(reinterpret_cast<const char*>(payload.data()), static_cast<std::streamsize>(payload.size()));
			return 0;
		}
		if (mode == "pack")
		{
			if (qmm_device_count() == 0)
			{
				std::puts("SKIP no CUDA device");
				return 77;
			}
			const PackedWeight w = GGUF::LoadPackedWeight(archive, t.name, CUDA{ 0 });
			const std::size_t count = w.OutFeatures() * w.InFeatures();
			float* dev = nullptr;
			std::vector<float> host(count);
			if (cudaMalloc(reinterpret_cast<void**>(&dev), count * sizeof(float)) != cudaSuccess)
			{
				throw std::runtime_error("cudaMalloc failed");
			}
			Detail::Check(qmm_dequantize(w.Handle(), dev, nullptr), "dequantize");
			if (cudaMemcpy(host.data(), dev, count * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess)
			{
				throw std::runtime_error("cudaMemcpy failed");
			}
			cudaFree(dev);
			out.write(reinterpret_cast<const char*>(host.data()), static_cast<std::streamsize>(count * sizeof(float)));
			return 0;
		}
		if (mode == "dequant")
		{
			if (qmm_device_count() == 0)
			{
				std::puts("SKIP no CUDA device");
				return 77;
			}
			const auto values = GGUF::DequantizeOnDevice(archive, t.name, CUDA{ 0 });
			out.write(reinterpret_cast<const char*>(values.data()), static_cast<std::streamsize>(values.size() * sizeof(float)));
			return 0;
		}
		std::puts("unknown mode");
		return 2;
	}
	catch (const std::runtime_error& e)
	{
		std::printf("ERROR %s\n", e.what());
		return 3;
	}
}
