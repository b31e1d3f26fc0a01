// A Swift face for libmlxq with the shape of the engine's `Linear` (Sources/MLXEngine/Transformer.swift:15):
// construct from borrowed device tensors, then `encode` onto a CUDA stream.  Not compiled in this
// repository (no Swift toolchain); it documents the binding a maintainer would add.
import CMLXQ

public enum MLXQError: Error {
    case invalidFile(String), unsupported(String), missingTensor(String), outOfMemory(String), gpuFailure(String),
         invalidArgument(String), collective(String), timeout(String)

    static func from(_ status: Int32) -> MLXQError {
        let text = String(cString: mlxq_last_error())
        switch status {
        case 1: return .invalidFile(text)
        case 2: return .unsupported(text)
        case 3: return .missingTensor(text)
        case 4: return .outOfMemory(text)
        case 5: return .gpuFailure(text)
        case 7: return .collective(text)
        case 8: return .timeout(text)
        default: return .invalidArgument(text)
        }
    }
}

/// A borrowed view of device memory, like the engine's `Tensor` (GPU.swift:145-154).
public struct DeviceTensor {
    public var pointer: UnsafeRawPointer
    public var dtype: mlxq_dtype
    public var shape: [Int]
    public init(pointer: UnsafeRawPointer, dtype: mlxq_dtype, shape: [Int]) {
        self.pointer = pointer; self.dtype = dtype; self.shape = shape
    }
}

public final class QuantizedLinear {
    let handle: mlxq_linear_t
    public let inDim: Int
    public let outDim: Int
    public let bits: Int
    public let groupSize: Int

    public init(weight: DeviceTensor, scales: DeviceTensor?, biases: DeviceTensor?, bias: DeviceTensor?, inDim: Int,
                outDim: Int? = nil, name: String, device: Int32 = 0) throws {
        var d = mlxq_linear_desc()
        d.weight = weight.pointer
        d.weight_rows = Int64(weight.shape.count == 2 ? weight.shape[0] : 0)
        d.weight_cols = Int64(weight.shape.count == 2 ? weight.shape[1] : 0)
        d.scales = scales?.pointer
        d.biases = biases?.pointer
        d.scales_rows = Int64(scales?.shape.first ?? 0); d.scales_cols = Int64(scales?.shape.last ?? 0)
        d.biases_rows = Int64(biases?.shape.first ?? 0); d.biases_cols = Int64(biases?.shape.last ?? 0)
        d.bias = bias?.pointer
        d.bias_len = Int64(bias?.shape.first ?? 0)
        d.in_dim = Int64(inDim)
        d.expect_out = Int64(outDim ?? 0)
        d.scale_dtype = Int32((scales?.dtype ?? MLXQ_F16).rawValue)
        d.bias_dtype = Int32((bias?.dtype ?? MLXQ_F16).rawValue)
        d.device = device
        var h: mlxq_linear_t?
        let status = name.withCString { cname -> Int32 in
            d.name = cname
            return mlxq_linear_create(&d, &h)
        }
        guard status == 0, let handle = h else { throw MLXQError.from(status) }
        self.handle = handle
        self.inDim = Int(mlxq_linear_in_dim(handle)); self.outDim = Int(mlxq_linear_out_dim(handle))
        self.bits = Int(mlxq_linear_bits(handle)); self.groupSize = Int(mlxq_linear_group_size(handle))
    }

    deinit { mlxq_linear_destroy(handle) }

    /// y[t, :outDim] = x[t] . W^T (+ bias), enqueued on `stream` (Transformer.swift:272).
    public func encode(stream: UnsafeMutableRawPointer?, x: UnsafeRawPointer, xDType: mlxq_dtype, xStride: Int,
                       y: UnsafeMutableRawPointer, yDType: mlxq_dtype, yStride: Int, T: Int) throws {
        let status = mlxq_linear_forward(handle, stream, x, Int32(xDType.rawValue), Int64(xStride), y, Int32(yDType.rawValue),
                                         Int64(yStride), Int64(T))
        if status != 0 { throw MLXQError.from(status) }
    }

    public static func useGemm64(T: Int, outDim: Int) -> Bool { mlxq_use_gemm64(Int64(T), Int64(outDim)) != 0 }
}
