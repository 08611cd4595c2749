// LiteNN-facing C++ adapter over the C ABI in include/litenn_qmm.h.
//
// It mirrors, for the quantized-matmul path only, the names, argument meaning and
// error behaviour of LiteNN's own operator surface so that a maintainer can drop
// it behind DeviceTraits<CUDA>::DoBinaryOp:
//   - QuantizedBlockFormat / QuantizationScheme / QuantizationParams / BlockQuantization
//     (src/LiteNN/Quantization.h:19-76, 442-452) with identical enumerator values;
//   - DataType, BinaryOp (src/LiteNN/DType.h:17-30, src/LiteNN/Operators.h:33-49);
//   - ShapeView (src/LiteNN/Misc.h:99-148), CUDA{deviceIndex} and
//     CUDAExecutionOptions{stream, synchronize} (src/LiteNN/Device/CUDA.h:70-74);
//   - errors are std::runtime_error with a formatted message
//     (src/LiteNN/Device/CUDA.cpp:89-131); nothing returns codes.
// The header is self-contained C++17 (it also compiles as C++20/26); inside LiteNN
// the mirrored declarations are replaced by the real headers.
#pragma once

#include <cstddef>
#include <cstdint>
#include <memory>
#include <mutex>
#include <numeric>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/litenn_qmm.h"

namespace LiteNN
{
namespace B200
{
	enum class DataType
	{
		Float32,
		Float64,
		Int32,
		Int64,
		Bool,
		Float16,
		BFloat16,
		Float8E4M3,
		Float8E5M2,
		Int8,
		UInt8,
	};

	enum class BinaryOp
	{
		Add,
		Subtract,
		Multiply,
		Divide,
		MatMul,
	};

	enum class QuantizationScheme
	{
		Affine,
		Block,
	};

	// Same enumerator order, hence the same numeric values, as LiteNN::QuantizedBlockFormat.
	enum class QuantizedBlockFormat : std::uint32_t
	{
		Scalar,
		GGML_Q4_0,
		GGML_Q4_1,
		GGML_Q5_0,
		GGML_Q5_1,
		GGML_Q8_0,
		GGML_Q8_1,
		GGML_Q2_K,
		GGML_Q3_K,
		GGML_Q4_K,
		GGML_Q5_K,
		GGML_Q6_K,
		GGML_Q8_K,
	};

	static_assert(static_cast<int>(QuantizedBlockFormat::GGML_Q4_0) == QMM_FMT_Q4_0);
	static_assert(static_cast<int>(QuantizedBlockFormat::GGML_Q8_0) == QMM_FMT_Q8_0);
	static_assert(static_cast<int>(QuantizedBlockFormat::GGML_Q4_K) == QMM_FMT_Q4_K);
	static_assert(static_cast<int>(QuantizedBlockFormat::GGML_Q6_K) == QMM_FMT_Q6_K);

	struct QuantizationParams
	{
		QuantizationScheme scheme{ QuantizationScheme::Affine };
		QuantizedBlockFormat blockFormat{ QuantizedBlockFormat::Scalar };
		DataType storageType{ DataType::Int8 };
		DataType expressedType{ DataType::Float32 };
		std::vector<std::size_t> expressedShape;
	};

	inline QuantizationParams BlockQuantization(QuantizedBlockFormat format, std::vector<std::size_t> expressedShape,
	                                            DataType expressedType = DataType::Float32)
	{
		QuantizationParams p;
		p.scheme = QuantizationScheme::Block;
		p.blockFormat = format;
		p.storageType = DataType::UInt8;
		p.expressedType = expressedType;
		p.expressedShape = std::move(expressedShape);
		return p;
	}

	// Non-owning in LiteNN (a span); here it copies up to four extents so that a braced
	// list can be passed safely.
	struct ShapeView
	{
		std::size_t Dims[4]{};
		std::size_t Size{};

		ShapeView(std::initializer_list<std::size_t> dims)
		{
			Assign(dims.begin(), dims.size());
		}
		ShapeView(const std::vector<std::size_t>& dims)
		{
			Assign(dims.data(), dims.size());
		}
		std::size_t NumDim() const
		{
			return Size;
		}
		std::size_t operator[](std::size_t i) const
		{
			return Dims[i];
		}
		std::size_t NumElements() const
		{
			return std::accumulate(Dims, Dims + Size, std::size_t{ 1 }, std::multiplies<>{});
		}

	private:
		void Assign(const std::size_t* p, std::size_t n)
		{
			if (n > 4)
			{
				throw std::runtime_error("ShapeView: at most 4 dimensions on this path");
			}
			Size = n;
			for (std::size_t i = 0; i < n; ++i)
			{
				Dims[i] = p[i];
			}
		}
	};

	struct CUDA
	{
		int deviceIndex{};
	};

	struct CUDAExecutionOptions
	{
		void* stream{};
		bool synchronize{ true };
	};

	namespace Detail
	{
		inline void Check(int status, const char* what)
		{
			if (status != QMM_OK)
			{
				throw std::runtime_error(std::string(what) + ": " + qmm_last_error());
			}
		}
	} // namespace Detail

	// A quantized weight resident on one GPU in the repacked tile layout.  Built once
	// from the importer's UInt8 payload (what Variable::CreateQuantized holds,
	// src/LiteNN/Graph.h:496-508); it replaces both DequantizeGGMLVariable + Transpose
	// at lowering time and the per-run weight copy of Interpreter::Execute(VariableRefNode)
	// (src/LiteNN/Runtime/Interpreter.h:325-329).
	class PackedWeight
	{
	public:
		PackedWeight() = default;

		PackedWeight(CUDA device, const QuantizationParams& params, const void* payload, std::size_t payloadBytes,
		             bool payloadOnDevice = false, CUDAExecutionOptions options = {})
		{
			if (params.scheme != QuantizationScheme::Block)
			{
				throw std::runtime_error("quantized MatMul requires block quantization");
			}
			if (params.storageType != DataType::UInt8)
			{
				throw std::runtime_error("block payload must be stored as UInt8 bytes");
			}
			if (params.expressedShape.size() != 2)
			{
				throw std::runtime_error("quantized MatMul weight must have a 2-D expressed shape [out, in]");
			}
			qmm_weight* raw = nullptr;
			Detail::Check(qmm_weight_create(device.deviceIndex, static_cast<int>(params.blockFormat), payload,
			                                payloadBytes, payloadOnDevice ? 1 : 0,
			                                static_cast<std::int64_t>(params.expressedShape[0]),
			                                static_cast<std::int64_t>(params.expressedShape[1]), options.stream, &raw),
			              "PackedWeight");
			handle_.reset(raw, [](qmm_weight* w) { qmm_weight_destroy(w); });
			outFeatures_ = params.expressedShape[0];
			inFeatures_ = params.expressedShape[1];
			device_ = device;
		}

		explicit operator bool() const
		{
			return static_cast<bool>(handle_);
		}
		const qmm_weight* Handle() const
		{
			return handle_.get();
		}
		std::size_t InFeatures() const
		{
			return inFeatures_;
		}
		std::size_t OutFeatures() const
		{
			return outFeatures_;
		}
		CUDA Device() const
		{
			return device_;
		}

	private:
		std::shared_ptr<qmm_weight> handle_;
		std::size_t inFeatures_{};
		std::size_t outFeatures_{};
		CUDA device_{};
	};

	// dst[M,N] = src1[M,K] x dequant(weight)[N,K]^T.  Shape and type checks follow
	// BinaryOpTraits<MatMul> (src/LiteNN/Operators.h:197-222): both operands 2-D,
	// src1.shape[1] == K, result dtype == input dtype.  Float32 activations of up to 16 rows
	// go to the dequant-fused GEMV; more rows (LiteNN's fp32 prefill lowering,
	// tools/gguf/LLaMABuilder.cpp:502-557) and BFloat16 activations go to the tcgen05 GEMM.
	inline void DoQuantizedMatMul(CUDA& device, void* dst, DataType type1, ShapeView shape1, const void* src1,
	                              const PackedWeight& weight, CUDAExecutionOptions options = {})
	{
		if (!weight)
		{
			throw std::runtime_error("quantized MatMul: weight is not packed");
		}
		if (weight.Device().deviceIndex != device.deviceIndex)
		{
			throw std::runtime_error("quantized MatMul: weight lives on another CUDA device");
		}
		if (shape1.NumDim() != 2)
		{
			throw std::runtime_error("MatMul requires 2-D operands");
		}
		if (shape1[1] != weight.InFeatures())
		{
			throw std::runtime_error("MatMul inner dimensions do not match");
		}
		const auto m = shape1[0];
		if (type1 == DataType::Float32)
		{
			if (m > QMM_GEMV_MAX_BATCH)
			{
				Detail::Check(qmm_gemm_f32(weight.Handle(), static_cast<const float*>(src1), static_cast<float*>(dst),
				                           static_cast<std::int64_t>(m), options.stream),
				              "quantized MatMul");
			}
			else
			{
				Detail::Check(qmm_gemv_f32(weight.Handle(), static_cast<const float*>(src1), static_cast<float*>(dst),
				                           static_cast<int>(m), options.stream),
				              "quantized MatMul");
			}
		}
		else if (type1 == DataType::BFloat16)
		{
			Detail::Check(qmm_gemm_bf16(weight.Handle(), src1, dst, static_cast<std::int64_t>(m), QMM_OUT_BF16,
			                            options.stream),
			              "quantized MatMul");
		}
		else
		{
			throw std::runtime_error("quantized MatMul supports Float32 and BFloat16 activations");
		}
		if (options.synchronize)
		{
			Detail::Check(qmm_stream_synchronize(device.deviceIndex, options.stream), "quantized MatMul");
			int status = 0;
			Detail::Check(qmm_kernel_status(device.deviceIndex, &status), "quantized MatMul");
		}
	}

	// The DoBinaryOp-shaped entry (src/LiteNN/Device/CUDA.h:150-154) for the fused graph
	// pattern payload(UInt8) -> DequantizeNode{Block,[N,K],Float32} -> Transpose -> MatMul:
	// src2 is the host payload of the quantized Variable, described by `params`.  Packed
	// weights are cached, so the repack and the upload happen once per weight, not once per
	// run.  An entry is identified by the device, the payload's address AND its byte count,
	// block format and expressed shape: a buffer whose address is reused for another tensor
	// is packed anew.  The payload must stay unchanged while its entry lives; call
	// Invalidate(payload) before rewriting or freeing a buffer whose successor at the same
	// address could have the same size, format and shape.
	class QuantizedMatMulCache
	{
	public:
		void DoBinaryOp(CUDA& device, BinaryOp op, void* dst, DataType type1, ShapeView shape1, const void* src1,
		                DataType type2, ShapeView shape2, const void* src2, const QuantizationParams& params,
		                CUDAExecutionOptions options = {})
		{
			if (op != BinaryOp::MatMul)
			{
				throw std::runtime_error("only MatMul takes a block-quantized operand");
			}
			if (type2 != DataType::UInt8 || shape2.NumDim() != 1)
			{
				throw std::runtime_error("block payload must be a 1-D UInt8 tensor");
			}
			const PackedWeight w = Get(device, params, src2, shape2.NumElements(), options);
			DoQuantizedMatMul(device, dst, type1, shape1, src1, w, options);
		}

		// Returns a handle that shares ownership, so it stays valid if the entry is invalidated meanwhile.
		PackedWeight Get(CUDA device, const QuantizationParams& params, const void* payload, std::size_t payloadBytes,
		                 CUDAExecutionOptions options = {})
		{
			std::lock_guard<std::mutex> lock(mutex_);
			Key key;
			key.device = device.deviceIndex;
			key.payload = payload;
			key.bytes = payloadBytes;
			key.format = static_cast<std::uint32_t>(params.blockFormat);
			key.rows = params.expressedShape.size() > 0 ? params.expressedShape[0] : 0;
			key.cols = params.expressedShape.size() > 1 ? params.expressedShape[1] : 0;
			auto it = cache_.find(key);
			if (it == cache_.end())
			{
				it = cache_.emplace(key, PackedWeight(device, params, payload, payloadBytes, false, options)).first;
			}
			return it->second;
		}

		// Drops every entry built from this payload address (on any device); returns how many.
		std::size_t Invalidate(const void* payload)
		{
			std::lock_guard<std::mutex> lock(mutex_);
			std::size_t dropped = 0;
			for (auto it = cache_.begin(); it != cache_.end();)
			{
				if (it->first.payload == payload)
				{
					it = cache_.erase(it);
					++dropped;
				}
				else
				{
					++it;
				}
			}
			return dropped;
		}

		std::size_t Size()
		{
			std::lock_guard<std::mutex> lock(mutex_);
			return cache_.size();
		}

		void Clear()
		{
			std::lock_guard<std::mutex> lock(mutex_);
			cache_.clear();
		}

	private:
		struct Key
		{
			int device{};
			const void* payload{};
			std::size_t bytes{};
			std::uint32_t format{};
			std::size_t rows{};
			std::size_t cols{};
			bool operator==(const Key& o) const
			{
				return device == o.device && payload == o.payload && bytes == o.bytes && format == o.format &&
				       rows == o.rows && cols == o.cols;
			}
		};
		struct KeyHash
		{
			std::size_t operator()(const Key& k) const
			{
				std::size_t h = std::hash<const void*>{}(k.payload);
				for (std::size_t v : { static_cast<std::size_t>(k.device), k.bytes, static_cast<std::size_t>(k.format), k.rows,
				                       k.cols })
				{
					h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
				}
				return h;
			}
		};
		std::mutex mutex_;
		std::unordered_map<Key, PackedWeight, KeyHash> cache_;
	};
} // namespace B200
} // namespace LiteNN
