// The two places a LiteNN runtime meets the block-quantized MatMul, restated as a small
// stand-alone C++17 runtime so that the pattern can be EXECUTED here (the reference itself
// needs a C++26 compiler and is not built in this tree):
//
//  * NodeLoop            - walks the nodes of one subgraph in id order, one output slot list
//                          per node, errors re-thrown with the failing node's id and kind, as
//                          Interpreter::RunSubgraphUnchecked does
//                          (src/LiteNN/Runtime/Interpreter.h:79-114).  It executes the pattern
//                          the validator already accepts but the reference throws on
//                          (Interpreter.h:380-391):
//                              VariableRef(UInt8 payload) -> Dequantize{Block,[N,K]} -> Transpose -> MatMul(x, .)
//                          A Block Dequantize yields a LAZY value (payload + parameters, nothing
//                          materialised); Transpose of a lazy value flips a flag; MatMul with a
//                          lazy transposed right operand goes to QuantizedMatMulCache::DoBinaryOp,
//                          so the weight is packed on its first use and stays resident on the GPU
//                          instead of being copied on every run (Interpreter.h:325-329).  A lazy
//                          value that reaches a result is materialised by qmm_dequantize.
//
//  * LibraryCallModule   - the compiled-payload side: kernel records whose name selects a library
//                          call, three pointer arguments (output, lhs, rhs) and three u32 scalars
//                          m, k, n, as RunCUDANativeLibraryCall reads them
//                          (src/LiteNN/Compiler/CompiledModule.cpp:4114-4180; record types
//                          Compiler/CUDANativePayload.h:95-123).  New kernel names
//                          litenn_qmatmul_{q4_0,q8_0,q4_k,q6_k}: rhs is a ConstantTensor range of
//                          the payload's constant data holding the GGUF bytes of W[N,K]; Load()
//                          packs every such range once (the reference uploads constantData once at
//                          Load, CompiledModule.cpp:4808-4809), Run() only launches.  The payload
//                          must carry kFeatureQuantizedMatMul, a bit above the reference's mask
//                          (CUDANativePayload.h:29-86), or Load() refuses it like any unknown bit.
#pragma once

#include <cuda_runtime_api.h>

#include <cstring>
#include <map>
#include <optional>
#include <sstream>
#include <string>
#include <string_view>
#include <variant>
#include <vector>

#include "LiteNNQuantMatMul.hpp"

namespace LiteNN
{
namespace B200
{
	namespace Runtime
	{
		// ---- device tensors -------------------------------------------------------------------------
		// Owns its allocation like Tensor<CUDA> (cudaMalloc / cudaFree per tensor, src/LiteNN/Device/CUDA.cpp:1753-1771).
		class DeviceTensor
		{
		public:
			DeviceTensor() = default;
			DeviceTensor(std::vector<std::size_t> shape, DataType dtype, CUDA device) : shape_(std::move(shape)), dtype_(dtype)
			{
				std::size_t bytes = ElementBytes(dtype);
				for (const auto d : shape_)
				{
					bytes *= d;
				}
				bytes_ = bytes;
				int previous = 0;
				cudaGetDevice(&previous);
				cudaSetDevice(device.deviceIndex);
				void* p = nullptr;
				const auto err = cudaMalloc(&p, bytes ? bytes : 1);
				cudaSetDevice(previous);
				if (err != cudaSuccess)
				{
					throw std::runtime_error(std::string("cudaMalloc failed: ") + cudaGetErrorString(err));
				}
				data_ = std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
			}
			static std::size_t ElementBytes(DataType t)
			{
				switch (t)
				{
				case DataType::Float32:
					return 4;
				case DataType::BFloat16:
				case DataType::Float16:
					return 2;
				case DataType::UInt8:
				case DataType::Int8:
					return 1;
				default:
					throw std::runtime_error("DeviceTensor: element type not used on this path");
				}
			}
			static DeviceTensor FromHost(const void* host, std::vector<std::size_t> shape, DataType dtype, CUDA device)
			{
				DeviceTensor t(std::move(shape), dtype, device);
				if (cudaMemcpy(t.RawData(), host, t.Bytes(), cudaMemcpyHostToDevice) != cudaSuccess)
				{
					throw std::runtime_error("cudaMemcpy to device failed");
				}
				return t;
			}
			void ToHost(void* host) const
			{
				if (cudaMemcpy(host, RawData(), bytes_, cudaMemcpyDeviceToHost) != cudaSuccess)
				{
					throw std::runtime_error("cudaMemcpy to host failed");
				}
			}
			void* RawData() const
			{
				return data_.get();
			}
			const std::vector<std::size_t>& Shape() const
			{
				return shape_;
			}
			DataType DType() const
			{
				return dtype_;
			}
			std::size_t Bytes() const
			{
				return bytes_;
			}

		private:
			std::shared_ptr<void> data_;
			std::vector<std::size_t> shape_;
			DataType dtype_{ DataType::Float32 };
			std::size_t bytes_{};
		};

		// ---- the node loop --------------------------------------------------------------------------
		struct NodeOutput
		{
			std::size_t node{};
			std::size_t port{};
		};

		// A graph variable: host bytes plus, for a quantized one, its parameters (Variable::CreateQuantized,
		// src/LiteNN/Graph.h:496-508).
		struct Variable
		{
			std::string name;
			DataType dtype{ DataType::Float32 };
			std::vector<std::size_t> shape;
			std::vector<std::uint8_t> bytes;
			std::optional<QuantizationParams> quantization;
		};

		struct ParamRefNode
		{
			std::size_t paramIndex{};
		};
		struct VariableRefNode
		{
			std::size_t variableIndex{};
		};
		struct DequantizeNode
		{
			NodeOutput input;
			QuantizationParams params;
			DataType targetType{ DataType::Float32 };
		};
		struct TransposeNode
		{
			NodeOutput input;
		};
		struct BinaryOpNode
		{
			BinaryOp op{ BinaryOp::MatMul };
			NodeOutput lhs;
			NodeOutput rhs;
		};
		using Node = std::variant<ParamRefNode, VariableRefNode, DequantizeNode, TransposeNode, BinaryOpNode>;

		inline const char* NodeKindName(const Node& node)
		{
			static const char* const names[] = { "ParamRefNode", "VariableRefNode", "DequantizeNode", "TransposeNode",
				                                 "BinaryOpNode" };
			return names[node.index()];
		}

		struct Subgraph
		{
			std::vector<Node> nodes;
			std::vector<NodeOutput> results;
		};

		struct Graph
		{
			std::vector<Variable> variables;
			Subgraph forward;
		};

		// What a slot holds: a device tensor, or a block-quantized weight that has not been (and on
		// the MatMul path never is) expanded to fp32.
		struct LazyQuantized
		{
			const Variable* variable{};
			QuantizationParams params;
			bool transposed{};
		};
		using Value = std::variant<DeviceTensor, LazyQuantized>;

		class NodeLoop
		{
		public:
			explicit NodeLoop(CUDA device = {}) : device_(device)
			{
			}

			std::vector<DeviceTensor> Run(const Graph& graph, const std::vector<DeviceTensor>& inputs)
			{
				const auto& subgraph = graph.forward;
				std::vector<std::vector<Value>> slots(subgraph.nodes.size());
				for (std::size_t id = 0; id < subgraph.nodes.size(); ++id)
				{
					try
					{
						std::visit([&](const auto& node) { Execute(graph, id, node, slots, inputs); }, subgraph.nodes[id]);
					}
					catch (const std::exception& ex)
					{
						std::ostringstream msg;
						msg << "Interpreter failed at subgraph 0, node " << id << " (" << NodeKindName(subgraph.nodes[id])
						    << "): " << ex.what();
						throw std::runtime_error(msg.str());
					}
				}
				std::vector<DeviceTensor> results;
				for (const auto& out : subgraph.results)
				{
					results.push_back(Materialize(Get(slots, out)));
				}
				return results;
			}

			// Packed weights built so far: one per quantized variable however many runs were made.
			std::size_t ResidentWeights()
			{
				return cache_.Size();
			}
			// Bytes copied host to device for variables during Run calls (0 for the quantized pattern after
			// its first use; the reference copies the whole variable per run).
			std::size_t VariableBytesCopied() const
			{
				return variableBytesCopied_;
			}

		private:
			static const Value& Get(const std::vector<std::vector<Value>>& slots, NodeOutput out)
			{
				if (out.node >= slots.size() || out.port >= slots[out.node].size())
				{
					throw std::runtime_error("node input refers to a value that has not been produced");
				}
				return slots[out.node][out.port];
			}

			void Execute(const Graph&, std::size_t id, const ParamRefNode& node, std::vector<std::vector<Value>>& slots,
			             const std::vector<DeviceTensor>& inputs)
			{
				if (node.paramIndex >= inputs.size())
				{
					throw std::runtime_error("RunSubgraph input count mismatch");
				}
				slots[id].push_back(inputs[node.paramIndex]);
			}

			void Execute(const Graph& graph, std::size_t id, const VariableRefNode& node, std::vector<std::vector<Value>>& slots,
			             const std::vector<DeviceTensor>&)
			{
				if (node.variableIndex >= graph.variables.size())
				{
					throw std::runtime_error("variable index out of range");
				}
				const auto& v = graph.variables[node.variableIndex];
				if (v.quantization && v.quantization->scheme == QuantizationScheme::Block)
				{
					// the payload stays on the host until a MatMul packs it; no per-run copy
					slots[id].push_back(LazyQuantized{ &v, *v.quantization, false });
					return;
				}
				variableBytesCopied_ += v.bytes.size();
				slots[id].push_back(DeviceTensor::FromHost(v.bytes.data(), v.shape, v.dtype, device_));
			}

			void Execute(const Graph&, std::size_t id, const DequantizeNode& node, std::vector<std::vector<Value>>& slots,
			             const std::vector<DeviceTensor>&)
			{
				const auto& in = Get(slots, node.input);
				const auto* lazy = std::get_if<LazyQuantized>(&in);
				if (node.params.scheme != QuantizationScheme::Block || lazy == nullptr)
				{
					throw std::runtime_error("DequantizeNode on this path takes a block-quantized variable");
				}
				if (node.targetType != DataType::Float32)
				{
					throw std::runtime_error("Block DequantizeNode produces Float32");
				}
				if (node.params.blockFormat != lazy->params.blockFormat || node.params.expressedShape != lazy->params.expressedShape)
				{
					throw std::runtime_error("DequantizeNode parameters do not match the variable's quantization");
				}
				slots[id].push_back(LazyQuantized{ lazy->variable, node.params, false });
			}

			void Execute(const Graph&, std::size_t id, const TransposeNode& node, std::vector<std::vector<Value>>& slots,
			             const std::vector<DeviceTensor>&)
			{
				const auto& in = Get(slots, node.input);
				const auto* lazy = std::get_if<LazyQuantized>(&in);
				if (lazy == nullptr)
				{
					throw std::runtime_error("TransposeNode of a dense tensor is outside this path");
				}
				if (lazy->params.expressedShape.size() != 2)
				{
					throw std::runtime_error("Transpose requires a 2-D operand");
				}
				LazyQuantized flipped = *lazy;
				flipped.transposed = !flipped.transposed;
				slots[id].push_back(flipped);
			}

			void Execute(const Graph&, std::size_t id, const BinaryOpNode& node, std::vector<std::vector<Value>>& slots,
			             const std::vector<DeviceTensor>&)
			{
				const auto& lhs = Get(slots, node.lhs);
				const auto& rhs = Get(slots, node.rhs);
				const auto* x = std::get_if<DeviceTensor>(&lhs);
				const auto* w = std::get_if<LazyQuantized>(&rhs);
				if (node.op != BinaryOp::MatMul || x == nullptr || w == nullptr)
				{
					throw std::runtime_error("only MatMul(dense, transposed block-quantized weight) runs on this path");
				}
				if (!w->transposed)
				{
					// MatMul(x[M,K], W[N,K]) without the transpose is a shape error unless N == K; refuse it either
					// way, because the kernels contract along the stored row (K) only.
					throw std::runtime_error("MatMul inner dimensions do not match (quantized weight is not transposed)");
				}
				if (x->Shape().size() != 2)
				{
					throw std::runtime_error("MatMul requires 2-D operands");
				}
				const std::size_t m = x->Shape()[0], n = w->params.expressedShape[0];
				DeviceTensor out({ m, n }, x->DType(), device_);
				cache_.DoBinaryOp(device_, BinaryOp::MatMul, out.RawData(), x->DType(), ShapeView(x->Shape()), x->RawData(),
				                  DataType::UInt8, ShapeView{ w->variable->bytes.size() }, w->variable->bytes.data(), w->params);
				slots[id].push_back(std::move(out));
			}

			DeviceTensor Materialize(const Value& v)
			{
				if (const auto* t = std::get_if<DeviceTensor>(&v))
				{
					return *t;
				}
				const auto& lazy = std::get<LazyQuantized>(v);
				if (lazy.transposed)
				{
					throw std::runtime_error("a transposed quantized weight is only consumed by MatMul");
				}
				const PackedWeight w = cache_.Get(device_, lazy.params, lazy.variable->bytes.data(), lazy.variable->bytes.size());
				DeviceTensor out(lazy.params.expressedShape, DataType::Float32, device_);
				Detail::Check(qmm_dequantize(w.Handle(), static_cast<float*>(out.RawData()), nullptr), "DequantizeNode");
				Detail::Check(qmm_stream_synchronize(device_.deviceIndex, nullptr), "DequantizeNode");
				return out;
			}

			CUDA device_;
			QuantizedMatMulCache cache_;
			std::size_t variableBytesCopied_{};
		};

		// ---- library calls of a compiled payload --------------------------------------------------------
		enum class ArgumentKind : std::uint32_t
		{
			InputTensor,
			OutputTensor,
			Workspace,
			Scalar,
			ConstantTensor,
		};

		struct ArgumentSpec
		{
			ArgumentKind kind{ ArgumentKind::InputTensor };
			std::uint32_t index{};
			std::uint64_t byteOffset{};
			std::uint64_t byteSize{};
		};

		struct KernelSpec
		{
			std::string name;
			std::vector<ArgumentSpec> arguments;
		};

		// One bit above every flag the reference defines today.
		constexpr std::uint64_t kFeatureQuantizedMatMul = 1ull << 40;

		struct InstructionPayload
		{
			std::uint64_t featureFlags{};
			std::vector<std::uint8_t> scalarData;
			std::vector<std::uint8_t> constantData;
			std::vector<KernelSpec> kernels;
		};

		inline std::optional<QuantizedBlockFormat> QuantizedMatMulLibraryCallFormat(std::string_view name)
		{
			static const std::map<std::string_view, QuantizedBlockFormat> names = {
				{ "litenn_qmatmul_q4_0", QuantizedBlockFormat::GGML_Q4_0 },
				{ "litenn_qmatmul_q8_0", QuantizedBlockFormat::GGML_Q8_0 },
				{ "litenn_qmatmul_q4_k", QuantizedBlockFormat::GGML_Q4_K },
				{ "litenn_qmatmul_q6_k", QuantizedBlockFormat::GGML_Q6_K },
			};
			const auto it = names.find(name);
			return it == names.end() ? std::nullopt : std::optional(it->second);
		}

		class LibraryCallModule
		{
		public:
			// Validates every kernel record and packs the constant range of each quantized MatMul once.
			static LibraryCallModule Load(InstructionPayload payload, CUDA device = {})
			{
				if ((payload.featureFlags & ~kFeatureQuantizedMatMul) != 0)
				{
					throw std::runtime_error("CUDA native payload has unsupported feature flags");
				}
				LibraryCallModule module;
				module.device_ = device;
				module.payload_ = std::move(payload);
				for (const auto& kernel : module.payload_.kernels)
				{
					const auto format = QuantizedMatMulLibraryCallFormat(kernel.name);
					if (!format)
					{
						throw std::runtime_error("Unsupported CUDA native library call '" + kernel.name + "'");
					}
					if ((module.payload_.featureFlags & kFeatureQuantizedMatMul) == 0)
					{
						throw std::runtime_error("CUDA native payload uses a quantized MatMul without declaring the feature");
					}
					if (kernel.arguments.size() != 6)
					{
						throw std::runtime_error("CUDA native quantized MatMul expects 3 pointer args and m/k/n scalar args");
					}
					const auto& rhs = kernel.arguments[2];
					if (rhs.kind != ArgumentKind::ConstantTensor)
					{
						throw std::runtime_error("CUDA native quantized MatMul expects its weight in the constant data");
					}
					if (rhs.byteOffset > module.payload_.constantData.size() ||
					    rhs.byteSize > module.payload_.constantData.size() - rhs.byteOffset)
					{
						throw std::runtime_error("CUDA native constant argument is out of bounds");
					}
					const std::size_t k = module.ReadScalarU32(kernel.arguments[4]), n = module.ReadScalarU32(kernel.arguments[5]);
					const auto params = BlockQuantization(*format, { n, k });
					module.weights_.emplace_back(device, params, module.payload_.constantData.data() + rhs.byteOffset,
					                             static_cast<std::size_t>(rhs.byteSize));
				}
				return module;
			}

			void Run(const std::vector<DeviceTensor>& inputs, std::vector<DeviceTensor>& outputs, CUDAExecutionOptions options = {})
			{
				for (std::size_t i = 0; i < payload_.kernels.size(); ++i)
				{
					RunLibraryCall(payload_.kernels[i], weights_[i], inputs, outputs, options);
				}
			}

			std::size_t ResidentWeights() const
			{
				return weights_.size();
			}

		private:
			std::uint32_t ReadScalarU32(const ArgumentSpec& arg) const
			{
				if (arg.kind != ArgumentKind::Scalar || arg.byteSize != 4 || arg.byteOffset > payload_.scalarData.size() ||
				    payload_.scalarData.size() - arg.byteOffset < 4)
				{
					throw std::runtime_error("CUDA native expected a u32 scalar argument");
				}
				std::uint32_t v = 0;
				std::memcpy(&v, payload_.scalarData.data() + arg.byteOffset, 4);
				return v;
			}

			static void* TensorPointer(const ArgumentSpec& arg, const std::vector<DeviceTensor>& inputs,
			                           const std::vector<DeviceTensor>& outputs, std::size_t needBytes, const char* role)
			{
				const auto& list = arg.kind == ArgumentKind::InputTensor ? inputs : outputs;
				if ((arg.kind != ArgumentKind::InputTensor && arg.kind != ArgumentKind::OutputTensor) || arg.index >= list.size())
				{
					throw std::runtime_error(std::string("CUDA native expected a device pointer argument for ") + role);
				}
				const auto& t = list[arg.index];
				if (arg.byteOffset > t.Bytes() || t.Bytes() - arg.byteOffset < needBytes)
				{
					throw std::runtime_error(std::string("CUDA native ") + role + " argument is out of bounds");
				}
				return static_cast<char*>(t.RawData()) + arg.byteOffset;
			}

			void RunLibraryCall(const KernelSpec& kernel, const PackedWeight& weight, const std::vector<DeviceTensor>& inputs,
			                    std::vector<DeviceTensor>& outputs, CUDAExecutionOptions options)
			{
				const std::size_t m = ReadScalarU32(kernel.arguments[3]), k = ReadScalarU32(kernel.arguments[4]),
				                  n = ReadScalarU32(kernel.arguments[5]);
				if (kernel.arguments[0].kind != ArgumentKind::OutputTensor || kernel.arguments[1].kind != ArgumentKind::InputTensor)
				{
					throw std::runtime_error("CUDA native quantized MatMul expects output, lhs input, constant rhs");
				}
				const DataType dtype = inputs.at(kernel.arguments[1].index).DType();
				const std::size_t eb = DeviceTensor::ElementBytes(dtype);
				void* out = TensorPointer(kernel.arguments[0], inputs, outputs, m * n * eb, "output");
				const void* lhs = TensorPointer(kernel.arguments[1], inputs, outputs, m * k * eb, "lhs");
				DoQuantizedMatMul(device_, out, dtype, ShapeView{ m, k }, lhs, weight, options);
			}

			CUDA device_;
			InstructionPayload payload_;
			std::vector<PackedWeight> weights_;
		};
	} // namespace Runtime
} // namespace B200
} // namespace LiteNN
