// GGUF archive reader without ggml: header, metadata key/values and tensor directory parsed
// from the published GGUF v2/v3 container layout, tensor payloads read on demand.
//
// It stands where LiteNN's importer calls into ggml today — gguf_init_from_file and the
// ggml_tensor accessors (tools/gguf/GGUFImporter.cpp:189-221), the metadata conversion
// (:340-446) and ImportTensor (:448-502) — and keeps that code's conventions:
//   - a tensor's shape is the reversed ggml `ne` (outermost dimension first), so a linear weight
//     reads [out_features, in_features] and quant blocks run along the last dimension;
//   - block-quantized tensors stay opaque byte payloads described by BlockQuantization(format,
//     shape, Float32); plain tensors keep their element type;
//   - the stored byte size must equal the size the type and shape imply ("inconsistent byte
//     size" otherwise); every failure is a std::runtime_error.
// LoadPackedWeight feeds a quantized tensor's payload straight into the upload-time repack
// (PackedWeight, LiteNNQuantMatMul.hpp), so the file-to-HBM path never dequantizes; DequantizeOnDevice
// is the fp32 route for tensors in a block format without matmul kernels.
#pragma once

#include <cuda_runtime_api.h>

#include <cstdint>
#include <cstring>
#include <fstream>
#include <map>
#include <optional>
#include <stdexcept>
#include <string>
#include <variant>
#include <vector>

#include "LiteNNQuantMatMul.hpp"

namespace LiteNN
{
namespace B200
{
namespace GGUF
{
	// Same alternatives as LiteNN::ModelMetadataValue for what GGUF can hold
	// (tools/gguf/GGUFImporter.cpp:340-435): scalars widen to 64 bits, arrays keep their element kind.
	using MetadataValue = std::variant<std::uint64_t, std::int64_t, double, bool, std::string, std::vector<std::uint64_t>,
	                                   std::vector<std::int64_t>, std::vector<double>, std::vector<bool>,
	                                   std::vector<std::string>>;

	struct MetadataEntry
	{
		std::string key;
		MetadataValue value;
	};

	// ggml_type ids as stored in a GGUF tensor directory.
	enum class TensorType : std::uint32_t
	{
		F32 = 0, F16 = 1, Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q8_1 = 9, Q2_K = 10, Q3_K = 11, Q4_K = 12,
		Q5_K = 13, Q6_K = 14, Q8_K = 15, I8 = 24, I16 = 25, I32 = 26, I64 = 27, F64 = 28, BF16 = 30,
	};

	struct TypeLayout
	{
		std::size_t blockElems;
		std::size_t blockBytes;
	};

	// Elements and bytes per block of every type the importer carries (plain types: one element).
	inline std::optional<TypeLayout> LayoutOf(TensorType t)
	{
		switch (t)
		{
		case TensorType::F32: return TypeLayout{ 1, 4 };
		case TensorType::F16: return TypeLayout{ 1, 2 };
		case TensorType::BF16: return TypeLayout{ 1, 2 };
		case TensorType::F64: return TypeLayout{ 1, 8 };
		case TensorType::I8: return TypeLayout{ 1, 1 };
		case TensorType::I16: return TypeLayout{ 1, 2 };
		case TensorType::I32: return TypeLayout{ 1, 4 };
		case TensorType::I64: return TypeLayout{ 1, 8 };
		case TensorType::Q4_0: return TypeLayout{ 32, 18 };
		case TensorType::Q4_1: return TypeLayout{ 32, 20 };
		case TensorType::Q5_0: return TypeLayout{ 32, 22 };
		case TensorType::Q5_1: return TypeLayout{ 32, 24 };
		case TensorType::Q8_0: return TypeLayout{ 32, 34 };
		case TensorType::Q8_1: return TypeLayout{ 32, 36 };
		case TensorType::Q2_K: return TypeLayout{ 256, 84 };
		case TensorType::Q3_K: return TypeLayout{ 256, 110 };
		case TensorType::Q4_K: return TypeLayout{ 256, 144 };
		case TensorType::Q5_K: return TypeLayout{ 256, 176 };
		case TensorType::Q6_K: return TypeLayout{ 256, 210 };
		case TensorType::Q8_K: return TypeLayout{ 256, 292 };
		default: return std::nullopt;
		}
	}

	// TryMapQuantizedBlockFormat (tools/gguf/GGUFImporter.cpp:257-304) for the formats above.
	inline std::optional<QuantizedBlockFormat> BlockFormatOf(TensorType t)
	{
		switch (t)
		{
		case TensorType::Q4_0: return QuantizedBlockFormat::GGML_Q4_0;
		case TensorType::Q4_1: return QuantizedBlockFormat::GGML_Q4_1;
		case TensorType::Q5_0: return QuantizedBlockFormat::GGML_Q5_0;
		case TensorType::Q5_1: return QuantizedBlockFormat::GGML_Q5_1;
		case TensorType::Q8_0: return QuantizedBlockFormat::GGML_Q8_0;
		case TensorType::Q8_1: return QuantizedBlockFormat::GGML_Q8_1;
		case TensorType::Q2_K: return QuantizedBlockFormat::GGML_Q2_K;
		case TensorType::Q3_K: return QuantizedBlockFormat::GGML_Q3_K;
		case TensorType::Q4_K: return QuantizedBlockFormat::GGML_Q4_K;
		case TensorType::Q5_K: return QuantizedBlockFormat::GGML_Q5_K;
		case TensorType::Q6_K: return QuantizedBlockFormat::GGML_Q6_K;
		case TensorType::Q8_K: return QuantizedBlockFormat::GGML_Q8_K;
		default: return std::nullopt;
		}
	}

	// TryMapPlainDataType (tools/gguf/GGUFImporter.cpp:233-255).
	inline std::optional<DataType> PlainTypeOf(TensorType t)
	{
		switch (t)
		{
		case TensorType::F32: return DataType::Float32;
		case TensorType::F64: return DataType::Float64;
		case TensorType::F16: return DataType::Float16;
		case TensorType::BF16: return DataType::BFloat16;
		case TensorType::I8: return DataType::Int8;
		case TensorType::I32: return DataType::Int32;
		case TensorType::I64: return DataType::Int64;
		default: return std::nullopt;
		}
	}

	struct TensorInfo
	{
		std::string name;
		std::vector<std::size_t> shape;  // outermost first (reversed ggml ne)
		TensorType type{};
		std::uint64_t offset{};          // from the start of the file
		std::size_t bytes{};
		std::optional<QuantizedBlockFormat> blockFormat;  // set for block-quantized tensors
		std::optional<DataType> plainType;                // set for plain tensors

		bool IsQuantized() const
		{
			return blockFormat.has_value();
		}
		// What Variable::CreateQuantized receives (tools/gguf/GGUFImporter.cpp:478-491).
		QuantizationParams Quantization() const
		{
			if (!blockFormat)
			{
				throw std::runtime_error("GGUF tensor '" + name + "' is not block-quantized");
			}
			return BlockQuantization(*blockFormat, shape, DataType::Float32);
		}
	};

	// LLaMAHyperparameters of tools/gguf/GGUFImporter.h:12-38, the fields this path uses.
	struct LLaMAHyperparameters
	{
		std::string architecture;
		std::size_t contextLength{};
		std::size_t embeddingLength{};
		std::size_t blockCount{};
		std::size_t feedForwardLength{};
		std::size_t attentionHeadCount{};
		std::size_t attentionHeadCountKV{};
		double rmsNormEpsilon{};
		double ropeFrequencyBase{ 10000.0 };
		std::size_t ropeDimensionCount{};

		std::size_t HeadDimension() const
		{
			return embeddingLength / attentionHeadCount;
		}
		std::size_t QueryGroupsPerKVHead() const
		{
			return attentionHeadCount / attentionHeadCountKV;
		}
	};

	class Archive
	{
	public:
		explicit Archive(const std::string& path) : path_(path), input_(path, std::ios::binary)
		{
			if (!input_)
			{
				throw std::runtime_error("Failed to open GGUF file '" + path + "'");
			}
			input_.seekg(0, std::ios::end);
			fileBytes_ = static_cast<std::uint64_t>(input_.tellg());
			input_.seekg(0);
			Parse();
		}

		std::uint32_t Version() const
		{
			return version_;
		}
		const std::vector<MetadataEntry>& Metadata() const
		{
			return metadata_;
		}
		const std::vector<TensorInfo>& Tensors() const
		{
			return tensors_;
		}

		const MetadataValue* FindMetadata(const std::string& key) const
		{
			for (const auto& e : metadata_)
			{
				if (e.key == key)
				{
					return &e.value;
				}
			}
			return nullptr;
		}

		const TensorInfo& Tensor(const std::string& name) const
		{
			const auto it = byName_.find(name);
			if (it == byName_.end())
			{
				throw std::runtime_error("GGUF archive has no tensor '" + name + "'");
			}
			return tensors_[it->second];
		}
		bool HasTensor(const std::string& name) const
		{
			return byName_.count(name) != 0;
		}

		// The tensor's bytes exactly as stored: the opaque UInt8 payload of a quantized Variable, or
		// the elements of a plain tensor.
		std::vector<std::uint8_t> ReadPayload(const TensorInfo& t)
		{
			std::vector<std::uint8_t> out(t.bytes);
			input_.clear();
			input_.seekg(static_cast<std::streamoff>(t.offset), std::ios::beg);
			if (!input_)
			{
				throw std::runtime_error("Failed to seek to GGUF data offset " + std::to_string(t.offset));
			}
			input_.read(reinterpret_cast<char*>(out.data()), static_cast<std::streamsize>(out.size()));
			if (static_cast<std::size_t>(input_.gcount()) != out.size())
			{
				throw std::runtime_error("Failed to read " + std::to_string(out.size()) + " bytes for GGUF tensor '" + t.name +
				                         "'");
			}
			return out;
		}

		// ParseLLaMAHyperparameters (tools/gguf/GGUFImporter.cpp:505-642) for `<arch>.*` keys.
		LLaMAHyperparameters ParseLLaMAHyperparameters() const
		{
			LLaMAHyperparameters h;
			h.architecture = String("general.architecture");
			const std::string p = h.architecture + ".";
			h.contextLength = Unsigned(p + "context_length");
			h.embeddingLength = Unsigned(p + "embedding_length");
			h.blockCount = Unsigned(p + "block_count");
			h.feedForwardLength = Unsigned(p + "feed_forward_length");
			h.attentionHeadCount = Unsigned(p + "attention.head_count");
			h.attentionHeadCountKV = FindMetadata(p + "attention.head_count_kv") ? Unsigned(p + "attention.head_count_kv")
			                                                                    : h.attentionHeadCount;
			h.rmsNormEpsilon = Real(p + "attention.layer_norm_rms_epsilon");
			if (FindMetadata(p + "rope.freq_base"))
			{
				h.ropeFrequencyBase = Real(p + "rope.freq_base");
			}
			if (h.attentionHeadCount == 0 || h.attentionHeadCountKV == 0 || h.embeddingLength % h.attentionHeadCount != 0 ||
			    h.attentionHeadCount % h.attentionHeadCountKV != 0)
			{
				throw std::runtime_error("GGUF LLaMA hyperparameters are inconsistent (head counts vs embedding length)");
			}
			h.ropeDimensionCount = FindMetadata(p + "rope.dimension_count") ? Unsigned(p + "rope.dimension_count")
			                                                               : h.HeadDimension();
			return h;
		}

	private:
		template <typename T>
		T Read()
		{
			T v{};
			input_.read(reinterpret_cast<char*>(&v), sizeof(T));
			if (static_cast<std::size_t>(input_.gcount()) != sizeof(T))
			{
				throw std::runtime_error("GGUF file '" + path_ + "' is truncated");
			}
			return v;
		}

		std::uint64_t ReadCount()
		{
			return version_ == 1 ? Read<std::uint32_t>() : Read<std::uint64_t>();
		}

		std::string ReadString()
		{
			const auto n = ReadCount();
			if (n > fileBytes_)
			{
				throw std::runtime_error("GGUF file '" + path_ + "' holds a string longer than the file");
			}
			std::string s(static_cast<std::size_t>(n), '\0');
			input_.read(s.data(), static_cast<std::streamsize>(n));
			if (static_cast<std::uint64_t>(input_.gcount()) != n)
			{
				throw std::runtime_error("GGUF file '" + path_ + "' is truncated");
			}
			return s;
		}

		MetadataValue ReadScalar(std::uint32_t type)
		{
			switch (type)
			{
			case 0: return static_cast<std::uint64_t>(Read<std::uint8_t>());
			case 1: return static_cast<std::int64_t>(Read<std::int8_t>());
			case 2: return static_cast<std::uint64_t>(Read<std::uint16_t>());
			case 3: return static_cast<std::int64_t>(Read<std::int16_t>());
			case 4: return static_cast<std::uint64_t>(Read<std::uint32_t>());
			case 5: return static_cast<std::int64_t>(Read<std::int32_t>());
			case 6: return static_cast<double>(Read<float>());
			case 7: return Read<std::uint8_t>() != 0;
			case 8: return ReadString();
			case 10: return Read<std::uint64_t>();
			case 11: return Read<std::int64_t>();
			case 12: return Read<double>();
			default: throw std::runtime_error("Unsupported GGUF metadata type " + std::to_string(type));
			}
		}

		template <typename Dst>
		std::vector<Dst> ReadArrayAs(std::uint32_t type, std::uint64_t count)
		{
			std::vector<Dst> out;
			out.reserve(static_cast<std::size_t>(count));
			for (std::uint64_t i = 0; i < count; ++i)
			{
				out.push_back(std::get<Dst>(ReadScalar(type)));
			}
			return out;
		}

		MetadataValue ReadValue(std::uint32_t type)
		{
			if (type != 9)
			{
				return ReadScalar(type);
			}
			const auto elem = Read<std::uint32_t>();
			const auto count = ReadCount();
			if (count > fileBytes_)
			{
				throw std::runtime_error("GGUF file '" + path_ + "' holds an array longer than the file");
			}
			switch (elem)
			{
			case 0: case 2: case 4: case 10: return ReadArrayAs<std::uint64_t>(elem, count);
			case 1: case 3: case 5: case 11: return ReadArrayAs<std::int64_t>(elem, count);
			case 6: case 12: return ReadArrayAs<double>(elem, count);
			case 7: return ReadArrayAs<bool>(elem, count);
			case 8: return ReadArrayAs<std::string>(elem, count);
			default: throw std::runtime_error("Unsupported GGUF metadata array type " + std::to_string(elem));
			}
		}

		void Parse()
		{
			char magic[4];
			input_.read(magic, 4);
			if (input_.gcount() != 4 || std::memcmp(magic, "GGUF", 4) != 0)
			{
				throw std::runtime_error("'" + path_ + "' is not a GGUF file (bad magic)");
			}
			version_ = Read<std::uint32_t>();
			if (version_ < 1 || version_ > 3)
			{
				throw std::runtime_error("Unsupported GGUF version " + std::to_string(version_));
			}
			const auto tensorCount = ReadCount();
			const auto kvCount = ReadCount();
			if (tensorCount > fileBytes_ || kvCount > fileBytes_)
			{
				throw std::runtime_error("GGUF file '" + path_ + "' has an implausible directory size");
			}
			metadata_.reserve(static_cast<std::size_t>(kvCount));
			for (std::uint64_t i = 0; i < kvCount; ++i)
			{
				std::string key = ReadString();
				const auto type = Read<std::uint32_t>();
				metadata_.push_back({ std::move(key), ReadValue(type) });
			}
			std::uint64_t alignment = 32;
			if (const auto* a = FindMetadata("general.alignment"))
			{
				if (const auto* u = std::get_if<std::uint64_t>(a))
				{
					alignment = *u;
				}
			}
			if (alignment == 0 || (alignment & (alignment - 1)) != 0)
			{
				throw std::runtime_error("GGUF general.alignment must be a power of two");
			}
			struct Raw
			{
				TensorInfo info;
				std::uint64_t relOffset;
			};
			std::vector<Raw> raw;
			raw.reserve(static_cast<std::size_t>(tensorCount));
			for (std::uint64_t i = 0; i < tensorCount; ++i)
			{
				Raw r;
				r.info.name = ReadString();
				const auto nDims = Read<std::uint32_t>();
				if (nDims == 0 || nDims > 4)
				{
					throw std::runtime_error("GGUF tensor '" + r.info.name + "' has an unsupported rank");
				}
				std::vector<std::uint64_t> ne(nDims);
				for (auto& d : ne)
				{
					d = ReadCount();
					if (d == 0)
					{
						throw std::runtime_error("GGUF tensor '" + r.info.name + "' has non-positive dimension 0");
					}
				}
				r.info.shape.assign(ne.rbegin(), ne.rend());  // TensorShape: outermost first
				r.info.type = static_cast<TensorType>(Read<std::uint32_t>());
				r.relOffset = Read<std::uint64_t>();
				const auto layout = LayoutOf(r.info.type);
				if (!layout)
				{
					throw std::runtime_error("Unsupported ggml tensor type " +
					                         std::to_string(static_cast<std::uint32_t>(r.info.type)) + " for tensor '" +
					                         r.info.name + "'");
				}
				if (ne[0] % layout->blockElems != 0)
				{
					throw std::runtime_error("GGUF tensor '" + r.info.name + "' row width " + std::to_string(ne[0]) +
					                         " is incompatible with ggml block size " + std::to_string(layout->blockElems));
				}
				std::size_t elems = 1;
				for (const auto d : ne)
				{
					elems *= static_cast<std::size_t>(d);
				}
				r.info.bytes = elems / layout->blockElems * layout->blockBytes;
				r.info.blockFormat = BlockFormatOf(r.info.type);
				r.info.plainType = PlainTypeOf(r.info.type);
				raw.push_back(std::move(r));
			}
			const auto dirEnd = static_cast<std::uint64_t>(input_.tellg());
			const auto dataStart = (dirEnd + alignment - 1) / alignment * alignment;
			for (std::size_t i = 0; i < raw.size(); ++i)
			{
				auto& r = raw[i];
				if (r.relOffset % alignment != 0)
				{
					throw std::runtime_error("GGUF tensor '" + r.info.name + "' is not aligned to general.alignment");
				}
				r.info.offset = dataStart + r.relOffset;
				// what the header implies for this tensor: up to the next tensor's offset or the end of the file
				std::uint64_t stored = fileBytes_ >= r.info.offset ? fileBytes_ - r.info.offset : 0;
				for (const auto& o : raw)
				{
					if (o.relOffset > r.relOffset && dataStart + o.relOffset - r.info.offset < stored)
					{
						stored = dataStart + o.relOffset - r.info.offset;
					}
				}
				if (stored < r.info.bytes)
				{
					throw std::runtime_error("GGUF tensor '" + r.info.name + "' has inconsistent byte size: header reports " +
					                         std::to_string(stored) + ", ggml metadata reports " + std::to_string(r.info.bytes));
				}
				byName_[r.info.name] = tensors_.size();
				tensors_.push_back(std::move(r.info));
			}
		}

		std::string String(const std::string& key) const
		{
			const auto* v = FindMetadata(key);
			const auto* s = v ? std::get_if<std::string>(v) : nullptr;
			if (!s)
			{
				throw std::runtime_error("GGUF metadata '" + key + "' is missing or not a string");
			}
			return *s;
		}
		std::size_t Unsigned(const std::string& key) const
		{
			const auto* v = FindMetadata(key);
			if (v)
			{
				if (const auto* u = std::get_if<std::uint64_t>(v))
				{
					return static_cast<std::size_t>(*u);
				}
				if (const auto* i = std::get_if<std::int64_t>(v))
				{
					if (*i >= 0)
					{
						return static_cast<std::size_t>(*i);
					}
				}
			}
			throw std::runtime_error("GGUF metadata '" + key + "' is missing or not a non-negative integer");
		}
		double Real(const std::string& key) const
		{
			const auto* v = FindMetadata(key);
			if (v)
			{
				if (const auto* d = std::get_if<double>(v))
				{
					return *d;
				}
				if (const auto* u = std::get_if<std::uint64_t>(v))
				{
					return static_cast<double>(*u);
				}
			}
			throw std::runtime_error("GGUF metadata '" + key + "' is missing or not a number");
		}

		std::string path_;
		std::ifstream input_;
		std::uint64_t fileBytes_{};
		std::uint32_t version_{};
		std::vector<MetadataEntry> metadata_;
		std::vector<TensorInfo> tensors_;
		std::map<std::string, std::size_t> byName_;
	};

	// File -> HBM: the payload of a quantized 2-D tensor goes straight into the upload-time repack.
	inline PackedWeight LoadPackedWeight(Archive& archive, const std::string& tensorName, CUDA device,
	                                     CUDAExecutionOptions options = {})
	{
		const auto& t = archive.Tensor(tensorName);
		const auto payload = archive.ReadPayload(t);
		return PackedWeight(device, t.Quantization(), payload.data(), payload.size(), false, options);
	}
	// File -> fp32 on the host through the GPU: what DequantizeGGMLVariable (tools/gguf/LLaMABuilder.cpp:66-162)
	// yields, for ANY block format the library knows, including those it has no matmul kernels for
	// (Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K).  The payload is uploaded as it is and dequantized on the device
	// (qmm_dequantize_raw), values bit-exact with ggml's to_float; rows = all leading dimensions folded.
	inline std::vector<float> DequantizeOnDevice(Archive& archive, const std::string& tensorName, CUDA device)
	{
		const auto& t = archive.Tensor(tensorName);
		if (!t.blockFormat || t.shape.empty())
		{
			throw std::runtime_error("GGUF tensor '" + tensorName + "' is not block-quantized");
		}
		const auto payload = archive.ReadPayload(t);
		const std::size_t k = t.shape.back();
		std::size_t rows = 1;
		for (std::size_t i = 0; i + 1 < t.shape.size(); ++i)
		{
			rows *= t.shape[i];
		}
		int previous = 0;
		cudaGetDevice(&previous);
		cudaSetDevice(device.deviceIndex);
		void* rawDev = nullptr;
		float* outDev = nullptr;
		std::vector<float> out(rows * k);
		const bool ok = cudaMalloc(&rawDev, payload.size()) == cudaSuccess &&
		                cudaMalloc(reinterpret_cast<void**>(&outDev), out.size() * sizeof(float)) == cudaSuccess &&
		                cudaMemcpy(rawDev, payload.data(), payload.size(), cudaMemcpyHostToDevice) == cudaSuccess;
		int status = ok ? qmm_dequantize_raw(device.deviceIndex, static_cast<int>(*t.blockFormat), rawDev,
		                                     static_cast<std::int64_t>(rows), static_cast<std::int64_t>(k), outDev, nullptr)
		                : QMM_E_CUDA;
		const std::string why = status != QMM_OK && ok ? qmm_last_error() : "device buffers";
		if (status == QMM_OK &&
		    cudaMemcpy(out.data(), outDev, out.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess)
		{
			status = QMM_E_CUDA;
		}
		cudaFree(rawDev);
		cudaFree(outDev);
		cudaSetDevice(previous);
		if (status != QMM_OK)
		{
			throw std::runtime_error("DequantizeOnDevice('" + tensorName + "'): " + why);
		}
		return out;
	}
} // namespace GGUF
} // namespace B200
} // namespace LiteNN
