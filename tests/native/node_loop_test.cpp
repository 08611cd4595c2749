// Executes the block-quantized MatMul pattern through the two runtime stand-ins of
// litenn_b200/host/QuantizedGraphRuntime.hpp, as a LiteNN runtime would:
//   (1) the node loop: VariableRef(UInt8) -> Dequantize{Block,[N,K]} -> Transpose -> MatMul(x, .), run twice
//       (weights must stay resident), plus a graph whose result is the dequantized weight itself;
//   (2) a compiled payload with one litenn_qmatmul_<fmt> library-call record (weight in the constant data,
//       m/k/n as u32 scalars), loaded once and run twice.
// Usage: node_loop_test <fmt> <n> <k> <m> <payload.bin> <x.bin> <expected_y.bin> <expected_w.bin>
// Prints "node_loop max_rel_err <v>", "dequant bit_exact <0|1>", "library_call max_rel_err <v>"; exit 0.
// Error behaviour is checked first and needs no GPU; without a device it then prints SKIP and exits 77.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>

#include "../../litenn_b200/host/QuantizedGraphRuntime.hpp"

using namespace LiteNN::B200;
using namespace LiteNN::B200::Runtime;

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

static double MaxRelErr(const std::vector<float>& got, const std::vector<float>& want)
{
	double max_e = 0, max_abs = 0;
	for (std::size_t i = 0; i < got.size(); ++i)
	{
		max_e = std::max(max_e, std::fabs(static_cast<double>(got[i]) - want[i]));
		max_abs = std::max(max_abs, std::fabs(static_cast<double>(want[i])));
	}
	return max_abs > 0 ? max_e / max_abs : max_e;
}

template <typename F>
static bool Throws(F&& f, const char* needle)
{
	try
	{
		f();
	}
	catch (const std::runtime_error& e)
	{
		if (std::string(e.what()).find(needle) != std::string::npos)
		{
			return true;
		}
		std::printf("FAIL: unexpected message: %s\n", e.what());
		return false;
	}
	std::printf("FAIL: no exception, expected '%s'\n", needle);
	return false;
}

static void PutU32(std::vector<std::uint8_t>& bytes, std::uint32_t v)
{
	const auto* p = reinterpret_cast<const std::uint8_t*>(&v);
	bytes.insert(bytes.end(), p, p + 4);
}

static InstructionPayload MakePayload(const char* kernelName, const std::vector<std::uint8_t>& weight, std::uint32_t m,
                                      std::uint32_t k, std::uint32_t n, std::uint64_t constantOffset)
{
	InstructionPayload p;
	p.featureFlags = kFeatureQuantizedMatMul;
	p.constantData.assign(constantOffset, 0xEE);   // another constant in front of the weight
	p.constantData.insert(p.constantData.end(), weight.begin(), weight.end());
	PutU32(p.scalarData, m);
	PutU32(p.scalarData, k);
	PutU32(p.scalarData, n);
	KernelSpec kernel;
	kernel.name = kernelName;
	kernel.arguments = { { ArgumentKind::OutputTensor, 0, 0, 0 },
		                 { ArgumentKind::InputTensor, 0, 0, 0 },
		                 { ArgumentKind::ConstantTensor, 0, constantOffset, weight.size() },
		                 { ArgumentKind::Scalar, 0, 0, 4 },
		                 { ArgumentKind::Scalar, 0, 4, 4 },
		                 { ArgumentKind::Scalar, 0, 8, 4 } };
	p.kernels.push_back(std::move(kernel));
	return p;
}

int main(int argc, char** argv)
{
	// ---- error behaviour: std::runtime_error, node id and kind in the node loop's message -------------------
	{
		std::vector<std::uint8_t> w(18);
		auto unknown = MakePayload("litenn_qmatmul_q9_9", w, 1, 32, 1, 0);
		auto noFlag = MakePayload("litenn_qmatmul_q4_0", w, 1, 32, 1, 0);
		noFlag.featureFlags = 0;
		auto otherFlag = MakePayload("litenn_qmatmul_q4_0", w, 1, 32, 1, 0);
		otherFlag.featureFlags |= 1ull << 50;
		auto beyond = MakePayload("litenn_qmatmul_q4_0", w, 1, 32, 1, 0);
		beyond.kernels[0].arguments[2].byteSize = 19;
		auto threeArgs = MakePayload("litenn_qmatmul_q4_0", w, 1, 32, 1, 0);
		threeArgs.kernels[0].arguments.resize(3);
		if (!Throws([&] { LibraryCallModule::Load(unknown); }, "Unsupported CUDA native library call 'litenn_qmatmul_q9_9'") ||
		    !Throws([&] { LibraryCallModule::Load(noFlag); }, "without declaring the feature") ||
		    !Throws([&] { LibraryCallModule::Load(otherFlag); }, "unsupported feature flags") ||
		    !Throws([&] { LibraryCallModule::Load(beyond); }, "out of bounds") ||
		    !Throws([&] { LibraryCallModule::Load(threeArgs); }, "expects 3 pointer args and m/k/n scalar args"))
		{
			return 1;
		}
		// a Dequantize whose input was never produced: the loop names the node
		Graph g;
		g.forward.nodes = { DequantizeNode{ { 5, 0 }, BlockQuantization(QuantizedBlockFormat::GGML_Q4_0, { 1, 32 }) } };
		NodeLoop loop;
		if (!Throws([&] { loop.Run(g, {}); }, "Interpreter failed at subgraph 0, node 0 (DequantizeNode)"))
		{
			return 1;
		}
	}
	if (qmm_device_count() == 0)
	{
		std::puts("SKIP no CUDA device");
		return 77;
	}
	if (argc != 9)
	{
		std::puts("usage: node_loop_test fmt n k m payload x expected_y expected_w");
		return 2;
	}
	try
	{
		const auto fmt = static_cast<QuantizedBlockFormat>(std::atoi(argv[1]));
		const std::size_t n = std::strtoull(argv[2], nullptr, 10), k = std::strtoull(argv[3], nullptr, 10),
		                  m = std::strtoull(argv[4], nullptr, 10);
		const auto payload = ReadAll<std::uint8_t>(argv[5]);
		const auto x = ReadAll<float>(argv[6]);
		const auto expectedY = ReadAll<float>(argv[7]);
		const auto expectedW = ReadAll<float>(argv[8]);
		CUDA device{ 0 };

		// ---- (1) node loop --------------------------------------------------------------------------------
		Graph graph;
		Variable weight;
		weight.name = "blk.0.ffn_up.weight";
		weight.dtype = DataType::UInt8;
		weight.shape = { payload.size() };
		weight.bytes = payload;
		weight.quantization = BlockQuantization(fmt, { n, k });
		graph.variables.push_back(weight);
		graph.forward.nodes = { ParamRefNode{ 0 },                                              // 0: x[M,K]
			                    VariableRefNode{ 0 },                                           // 1: payload
			                    DequantizeNode{ { 1, 0 }, *weight.quantization },               // 2: W[N,K]
			                    TransposeNode{ { 2, 0 } },                                      // 3: Wt[K,N]
			                    BinaryOpNode{ BinaryOp::MatMul, { 0, 0 }, { 3, 0 } } };         // 4: y[M,N]
		graph.forward.results = { { 4, 0 } };
		NodeLoop loop(device);
		const auto xDev = DeviceTensor::FromHost(x.data(), { m, k }, DataType::Float32, device);
		std::vector<float> y(m * n);
		for (int run = 0; run < 2; ++run)
		{
			const auto results = loop.Run(graph, { xDev });
			if (results.size() != 1 || results[0].Shape() != std::vector<std::size_t>{ m, n })
			{
				std::puts("FAIL: node loop result shape");
				return 1;
			}
			results[0].ToHost(y.data());
		}
		if (loop.ResidentWeights() != 1 || loop.VariableBytesCopied() != 0)
		{
			std::puts("FAIL: the weight was packed or copied again on the second run");
			return 1;
		}
		std::printf("node_loop max_rel_err %.3e\n", MaxRelErr(y, expectedY));

		// the dequantized weight as a graph result (materialised through the same packed weight)
		const Subgraph matmulForward = graph.forward;   // same Graph object: the variable (and its payload address) stays
		graph.forward.nodes.resize(3);
		graph.forward.results = { { 2, 0 } };
		const auto wDev = loop.Run(graph, { xDev });
		graph.forward = matmulForward;
		std::vector<float> wHost(n * k);
		wDev[0].ToHost(wHost.data());
		std::printf("dequant bit_exact %d\n", std::memcmp(wHost.data(), expectedW.data(), wHost.size() * 4) == 0 ? 1 : 0);
		if (loop.ResidentWeights() != 1)
		{
			std::puts("FAIL: dequantize built a second packed weight");
			return 1;
		}

		// MatMul against the untransposed weight, and a wrong inner dimension: errors carry the node
		Graph bad = graph;
		bad.forward.nodes[4] = BinaryOpNode{ BinaryOp::MatMul, { 0, 0 }, { 2, 0 } };
		if (!Throws([&] { loop.Run(bad, { xDev }); }, "node 4 (BinaryOpNode)"))
		{
			return 1;
		}
		const auto xWrong = DeviceTensor({ m, k + 32 }, DataType::Float32, device);
		if (!Throws([&] { loop.Run(graph, { xWrong }); }, "MatMul inner dimensions do not match"))
		{
			return 1;
		}

		// ---- (2) compiled payload with a library-call record ------------------------------------------------
		static const char* const names[] = { "", "litenn_qmatmul_q4_0", "", "", "", "litenn_qmatmul_q8_0", "", "", "",
			                                 "litenn_qmatmul_q4_k", "", "litenn_qmatmul_q6_k" };
		auto module = LibraryCallModule::Load(MakePayload(names[static_cast<int>(fmt)], payload, static_cast<std::uint32_t>(m),
		                                                  static_cast<std::uint32_t>(k), static_cast<std::uint32_t>(n), 64),
		                                      device);
		std::vector<DeviceTensor> outputs = { DeviceTensor({ m, n }, DataType::Float32, device) };
		std::vector<float> y2(m * n);
		for (int run = 0; run < 2; ++run)
		{
			module.Run({ xDev }, outputs);
			outputs[0].ToHost(y2.data());
		}
		if (module.ResidentWeights() != 1)
		{
			std::puts("FAIL: library-call module holds more than one weight");
			return 1;
		}
		std::printf("library_call max_rel_err %.3e\n", MaxRelErr(y2, expectedY));
		// an output tensor too small for m x n is refused before any launch
		std::vector<DeviceTensor> small = { DeviceTensor({ m, n - 1 }, DataType::Float32, device) };
		if (!Throws([&] { module.Run({ xDev }, small); }, "output argument is out of bounds"))
		{
			return 1;
		}
		return 0;
	}
	catch (const std::runtime_error& e)
	{
		std::printf("FAIL: %s\n", e.what());
		return 1;
	}
}
