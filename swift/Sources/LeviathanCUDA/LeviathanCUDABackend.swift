// NOT COMPILED HERE: this repository's image has no swift toolchain.  Written against
// include/leviathan_cuda.h; every call below names the reference interface it stands in for.
import CLeviathanCUDA
import Foundation

/// The typed errors of the reference's quantized backends (Q4Error, Sources/LeviathanCore/Q4.swift:17-31),
/// carried by name so that this file builds without LeviathanCore; inside LeviathanCore map them to Q4Error.
public enum LevCUDAError: Error, Equatable {
    case unavailable(String)
    case badDimensions(String)
    case wrongInputCount(Int, expected: Int)
    case nonFiniteInput(String)
    case nonFiniteScale
    case nonFiniteOutput
    case integerOverflow(String)
    case exceedsWorkload(String)
    case commandFailed(String)
}

/// Q4MatvecEvidence of the reference (Q4.swift:117-124), same fields.
public struct LevMatvecEvidence: Sendable {
    public let deviceName: String
    public let deviceMaxBufferLength: Int
    public let recommendedMaxWorkingSetSize: Int
    public let outDim: Int
    public let inDim: Int
    public let commandStatus: String
}

func levThrow(_ status: Int32, _ ctx: OpaquePointer?, xCount: Int = 0, inDim: Int = 0) throws {
    if status == 0 { return }
    let message = ctx.map { String(cString: lev_last_error($0)) } ?? String(cString: lev_status_name(status))
    switch lev_status(UInt32(status)) {
    case LEV_BAD_DIMENSIONS: throw LevCUDAError.badDimensions(message)
    case LEV_WRONG_INPUT_COUNT: throw LevCUDAError.wrongInputCount(xCount, expected: inDim)
    case LEV_NONFINITE_INPUT: throw LevCUDAError.nonFiniteInput("activation vector")
    case LEV_NONFINITE_SCALE: throw LevCUDAError.nonFiniteScale
    case LEV_NONFINITE_OUTPUT: throw LevCUDAError.nonFiniteOutput
    case LEV_INTEGER_OVERFLOW: throw LevCUDAError.integerOverflow(message)
    case LEV_EXCEEDS_WORKLOAD: throw LevCUDAError.exceedsWorkload(message)
    case LEV_DEVICE_UNAVAILABLE: throw LevCUDAError.unavailable(message)
    default: throw LevCUDAError.commandFailed(message)
    }
}

typealias HostMatvec = @convention(c) (OpaquePointer?, UnsafePointer<UInt8>?, Int, Int64, Int64,
                                       UnsafePointer<Float>?, Int64, UnsafeMutablePointer<Float>?,
                                       UnsafeMutablePointer<lev_evidence>?) -> Int32

func reporting(_ call: HostMatvec, blocks: [UInt8], outDim: Int, inDim: Int, x: [Float]) throws
        -> (output: [Float], evidence: LevMatvecEvidence) {
    var ctx: OpaquePointer?
    try levThrow(lev_cuda_init(0, &ctx), nil)
    defer { lev_cuda_destroy(ctx) }
    var y = [Float](repeating: 0, count: max(outDim, 0))
    var ev = lev_evidence()
    let st = blocks.withUnsafeBufferPointer { b in
        x.withUnsafeBufferPointer { xv in
            call(ctx, b.baseAddress, b.count, Int64(outDim), Int64(inDim), xv.baseAddress, Int64(xv.count), &y, &ev)
        }
    }
    try levThrow(st, ctx, xCount: x.count, inDim: inDim)
    let name = withUnsafePointer(to: &ev.device_name) {
        $0.withMemoryRebound(to: CChar.self, capacity: 128) { String(cString: $0) }
    }
    var hw = lev_hw_profile()
    _ = lev_cuda_hardware_profile(ctx, &hw)
    return (y, LevMatvecEvidence(deviceName: name, deviceMaxBufferLength: Int(hw.total_memory),
                                 recommendedMaxWorkingSetSize: Int(hw.free_memory),
                                 outDim: outDim, inDim: inDim, commandStatus: "completed"))
}

/// Q4MetalBackend.matvecReporting (Sources/LeviathanCore/Q4.swift:165-167): GGUF Q4_0 block bytes in host
/// memory, one activation vector, f32 output and the run's evidence.
public enum Q4CUDABackend {
    public static func matvecReporting(blocks: [UInt8], outDim: Int, inDim: Int, x: [Float]) throws
            -> (output: [Float], evidence: LevMatvecEvidence) {
        try reporting(lev_q4_0_matvec_host, blocks: blocks, outDim: outDim, inDim: inDim, x: x)
    }
}

/// Q6MetalBackend.matvecReporting (Sources/LeviathanCore/Q6.swift:199-201).
public enum Q6CUDABackend {
    public static func matvecReporting(blocks: [UInt8], outDim: Int, inDim: Int, x: [Float]) throws
            -> (output: [Float], evidence: LevMatvecEvidence) {
        try reporting(lev_q6_k_matvec_host, blocks: blocks, outDim: outDim, inDim: inDim, x: x)
    }
}

/// Resident weights and the per-token calls of Gemma4Runner (Gemma4.swift:2583-2631 for the upload,
/// :3611-3905 for the loop).  Activations stay in device buffers the caller owns (cudaMalloc through any
/// binding, or the pointers of another runtime); this type only sequences C-ABI calls on the context's stream.
public final class LevCUDARunner {
    public let ctx: OpaquePointer
    private var tensors: [String: OpaquePointer] = [:]
    private var experts: [Int: OpaquePointer] = [:]
    private let gguf: OpaquePointer

    /// GGUFFile(path:) + the resident copy (GGUF.swift:96-178): tensors are uploaded by name on first use.
    public init(modelPath: String, device: Int32 = 0) throws {
        var c: OpaquePointer?
        try levThrow(lev_cuda_init(device, &c), nil)
        ctx = c!
        var g: OpaquePointer?
        var err = [CChar](repeating: 0, count: 256)
        let st = lev_gguf_open(modelPath, &g, &err, err.count)
        guard st == 0, let file = g else {
            lev_cuda_destroy(ctx)
            throw LevCUDAError.commandFailed(String(cString: err))
        }
        gguf = file
    }

    deinit {
        for (_, w) in tensors { lev_weights_free(ctx, w) }
        for (_, m) in experts { lev_moe_weights_free(ctx, m) }
        lev_gguf_close(gguf)
        lev_cuda_destroy(ctx)
    }

    public func tensor(_ name: String) throws -> OpaquePointer {
        if let w = tensors[name] { return w }
        var w: OpaquePointer?
        try levThrow(lev_gguf_upload(ctx, gguf, name, &w), ctx)
        tensors[name] = w!
        return w!
    }

    public func moe(layer: Int) throws -> OpaquePointer {
        if let m = experts[layer] { return m }
        var m: OpaquePointer?
        try levThrow(lev_gguf_moe_upload(ctx, gguf, Int32(layer), 0, 0, &m, nil), ctx)
        experts[layer] = m!
        return m!
    }

    /// matvec(tensor:x:y:) of the runner (Gemma4.swift:2960-3050): y = W[rowOffset ..< rowOffset + rows] x.
    public func matvec(tensor name: String, rowOffset: Int = 0, rows: Int, x: UnsafePointer<Float>, xCount: Int,
                       y: UnsafeMutablePointer<Float>, yCapacity: Int) throws {
        try levThrow(lev_matvec(ctx, try tensor(name), Int64(rowOffset), Int64(rows), x, Int64(xCount), 1, y,
                                Int64(yCapacity), Int32(LEV_SCHEDULE_AUTO), 0), ctx, xCount: xCount)
    }

    /// decodeEmbedding (Gemma4.swift:3558-3578): tokens are device memory, scale = sqrt(hidden).
    public func embed(tokens: UnsafePointer<Int32>, count: Int, hidden: Int, into x: UnsafeMutablePointer<Float>) throws {
        try levThrow(lev_embed_rows(ctx, try tensor("token_embd.weight"), tokens, Int64(count),
                                    Float(Double(hidden).squareRoot()), x), ctx)
    }

    /// The routed experts of one layer (router scores, top-k, expert FFNs, ordered combine;
    /// Gemma4.swift:3794-3880) without the reference's per-layer readback.
    public func routedExperts(layer: Int, h: UnsafePointer<Float>, tokens: Int, topK: Int,
                              out: UnsafeMutablePointer<Float>) throws {
        try levThrow(lev_moe_layer(ctx, try moe(layer: layer), h, Int64(tokens), Int32(topK), out, nil, nil, 0), ctx)
    }

    /// The tail of forwardToken (Gemma4.swift:3622-3643): final norm folded into the head product, softcap,
    /// greedy argmax; the chosen ids stay on the device for the next embed call.
    public func head(x: UnsafePointer<Float>, hidden: Int, vocab: Int, normWeight: UnsafePointer<Float>,
                     logits: UnsafeMutablePointer<Float>, softcap: Float, token: UnsafeMutablePointer<Int32>) throws {
        var f = lev_fusion(prologue: Int32(LEV_PROLOGUE_RMSNORM), norm_weight: normWeight, eps: 1e-6, residual: nil, alpha: 0)
        try levThrow(lev_matvec_fused(ctx, try tensor("token_embd.weight"), 0, Int64(vocab), x, Int64(hidden), 1, &f,
                                      logits, Int64(vocab)), ctx)
        try levThrow(lev_softcap(ctx, logits, Int64(vocab), softcap), ctx)
        try levThrow(lev_argmax(ctx, logits, 1, Int64(vocab), token, nil), ctx)
    }

    public func synchronize() throws { try levThrow(lev_cuda_synchronize(ctx), ctx) }
}
