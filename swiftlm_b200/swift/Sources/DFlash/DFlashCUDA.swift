// DFlashCUDA.swift — the three DFlash kernel entry points on libdflash_cuda (B200, sm_100a).
//
// Added next to DFlashKernels.swift; DFlashKernels.swift.patch makes the public entry points
// (tapeReplayKernel, gatedDeltaKernelWithTape, batchedSDPA2Pass) forward here in place of their Metal
// bodies.  Signatures, argument meaning, output shapes and dtypes are those of
// Sources/DFlash/DFlashKernels.swift:252-258, :316-324 and :737-743, so RecurrentRollbackCache, the
// provider registered by the server and DFlashKernelBench keep compiling unchanged.
//
// Error behaviour: the reference's entry points never throw and never trap — an ineligible shape takes
// the array-ops statement (tapeReplayOps / gatedDeltaOpsWithTape, which run on whatever device the
// array library is on) and batchedSDPA2Pass returns nil.  The same holds here: every function below
// returns nil when the library answers anything but DFLASH_OK, leaves the status and message in
// DFlashCUDA.lastStatus / lastError, and the caller in DFlashKernels.swift continues exactly as the
// reference does for a missing kernel.  Nothing here aborts the process.
//
// Written against include/dflash_cuda.h without a Swift toolchain at hand: kept to plain calls so that a
// maintainer's first compile finds little to fix.  The one assumption about the array library is the
// CUDAArrayAccess protocol below.

import CDFlashCUDA
import Foundation
import MLX

/// What the CUDA backend of the array library has to expose for a dense, evaluated array: its device
/// address and the CUDA stream its producer was ordered on.  A maintainer conforms MLXArray to it in a
/// few lines next to the backend (the names on the right-hand side depend on that backend).
public protocol CUDAArrayAccess {
    /// Device address of element 0 of an evaluated, row-major contiguous array.
    var cudaDevicePointer: UnsafeMutableRawPointer { get }
}

/// The stream kernels are enqueued on.  Defaults to the legacy default stream (nil); a backend with its
/// own stream sets this once at start-up.
public enum DFlashCUDAStream {
    nonisolated(unsafe) public static var current: UnsafeMutableRawPointer? = nil
}

/// Scratch for the split-KV partials of the attention kernel: caller-owned as the C ABI wants it, grown on
/// demand, reused across calls on the same stream.
final class DFlashWorkspace {
    static let shared = DFlashWorkspace()
    private var buffer: MLXArray?
    private let lock = NSLock()
    func device(atLeast bytes: Int) -> (UnsafeMutableRawPointer?, Int) {
        lock.lock(); defer { lock.unlock() }
        if bytes == 0 { return (nil, 0) }
        if buffer == nil || buffer!.size < bytes {
            let b = MLXArray.zeros([bytes], dtype: .uint8)
            MLX.eval(b)
            buffer = b
        }
        return ((buffer! as! CUDAArrayAccess).cudaDevicePointer, buffer!.size)
    }
}

public enum DFlashCUDA {
    /// Status and message of the last call on this thread that did not return DFLASH_OK.
    nonisolated(unsafe) public private(set) static var lastStatus: Int32 = 0
    nonisolated(unsafe) public private(set) static var lastError: String = ""

    private static func dtypeCode(_ t: DType) -> Int32? {
        switch t {
        case .float32: return Int32(DFLASH_F32.rawValue)
        case .bfloat16: return Int32(DFLASH_BF16.rawValue)
        case .float16: return Int32(DFLASH_F16.rawValue)
        case .uint8, .bool: return Int32(DFLASH_U8.rawValue)
        default: return nil
        }
    }

    private static func ok(_ status: Int32) -> Bool {
        if status == 0 { return true }
        lastStatus = status
        lastError = String(cString: dflash_last_error_string())
        return false
    }

    /// Evaluated, contiguous copy of `a` in `dtype` (or its own dtype) and its device address.
    private static func dense(_ a: MLXArray, as dtype: DType? = nil) -> (MLXArray, UnsafeMutableRawPointer)? {
        let c = MLX.contiguous(dtype == nil || a.dtype == dtype! ? a : a.asType(dtype!))
        MLX.eval(c)
        guard let access = c as? CUDAArrayAccess else { return nil }
        return (c, access.cudaDevicePointer)
    }

    /// Fresh output array and its device address.
    private static func output(_ shape: [Int], _ dtype: DType) -> (MLXArray, UnsafeMutableRawPointer)? {
        let o = MLXArray.zeros(shape, dtype: dtype)
        MLX.eval(o)
        guard let access = o as? CUDAArrayAccess else { return nil }
        return (o, access.cudaDevicePointer)
    }

    // MARK: tape replay — Sources/DFlash/DFlashKernels.swift:252-301

    /// S <- S * g_t + delta_t (x) k_t over the T steps of `tape` (the caller has sliced the accepted
    /// steps, RecurrentRollbackCache.swift:115-118).  Returns the replayed state in fp32, or nil.
    public static func tapeReplay(tape: MLXArray, k: MLXArray, g: MLXArray, state: MLXArray,
                                  mask: MLXArray? = nil) -> MLXArray? {
        guard k.ndim == 4, tape.ndim == 4, state.ndim == 4, let kg = dtypeCode(k.dtype) else { return nil }
        let (B, T, Hk, Dk) = (k.dim(0), k.dim(1), k.dim(2), k.dim(3))
        let (Hv, Dv) = (tape.dim(2), tape.dim(3))
        guard let (tapeA, tapeP) = dense(tape, as: .float32), let (kA, kP) = dense(k),
              let (gA, gP) = dense(g, as: k.dtype), let (sA, sP) = dense(state, as: .float32),
              let (out, outP) = output(state.shape, .float32) else { return nil }
        var maskP: UnsafeMutableRawPointer? = nil
        var maskCode: Int32 = 0
        var maskA: MLXArray? = nil
        if let mask {
            guard let code = dtypeCode(mask.dtype), let (mA, mP) = dense(mask) else { return nil }
            (maskA, maskP, maskCode) = (mA, mP, code)
        }
        let st = dflash_tape_replay(tapeP.assumingMemoryBound(to: Float.self), kP, gP,
                                    sP.assumingMemoryBound(to: Float.self), maskP, nil,
                                    outP.assumingMemoryBound(to: Float.self),
                                    Int32(B), Int32(T), Int32(Hk), Int32(Hv), Int32(Dk), Int32(Dv),
                                    g.ndim == 4 ? 1 : 0, kg, maskCode, DFlashCUDAStream.current)
        withExtendedLifetime((tapeA, kA, gA, sA, maskA)) {}
        return ok(st) ? out : nil
    }

    // MARK: gated-delta forward with tape — Sources/DFlash/DFlashKernels.swift:316-367

    /// Returns (y in q's dtype, new state fp32, innovation tape fp32), or nil.
    public static func gatedDeltaWithTape(q: MLXArray, k: MLXArray, v: MLXArray, g: MLXArray, beta: MLXArray,
                                          state: MLXArray, mask: MLXArray? = nil) -> (MLXArray, MLXArray, MLXArray)? {
        guard q.ndim == 4, k.ndim == 4, v.ndim == 4, state.ndim == 4, let inCode = dtypeCode(q.dtype) else { return nil }
        let (B, T, Hk, Dk) = (k.dim(0), k.dim(1), k.dim(2), k.dim(3))
        let (Hv, Dv) = (v.dim(2), v.dim(3))
        guard let (qA, qP) = dense(q), let (kA, kP) = dense(k, as: q.dtype), let (vA, vP) = dense(v, as: q.dtype),
              let (gA, gP) = dense(g, as: q.dtype), let (bA, bP) = dense(beta, as: q.dtype),
              let (sA, sP) = dense(state, as: .float32),
              let (y, yP) = output([B, T, Hv, Dv], q.dtype), let (newState, nsP) = output(state.shape, .float32),
              let (tape, tapeP) = output([B, T, Hv, Dv], .float32) else { return nil }
        var maskP: UnsafeMutableRawPointer? = nil
        var maskCode: Int32 = 0
        var maskA: MLXArray? = nil
        if let mask {
            guard let code = dtypeCode(mask.dtype), let (mA, mP) = dense(mask) else { return nil }
            (maskA, maskP, maskCode) = (mA, mP, code)
        }
        let st = dflash_gated_delta_tape(qP, kP, vP, gP, bP, sP.assumingMemoryBound(to: Float.self), maskP, nil,
                                         yP, nsP.assumingMemoryBound(to: Float.self),
                                         tapeP.assumingMemoryBound(to: Float.self),
                                         Int32(B), Int32(T), Int32(Hk), Int32(Hv), Int32(Dk), Int32(Dv),
                                         g.ndim == 4 ? 1 : 0, inCode, maskCode, DFlashCUDAStream.current)
        withExtendedLifetime((qA, kA, vA, gA, bA, sA, maskA)) {}
        return ok(st) ? (y, newState, tape) : nil
    }

    // MARK: block-verify attention — Sources/DFlash/DFlashKernels.swift:737-815

    /// Returns the attention output in the input dtype, or nil exactly where the reference returns nil
    /// (query length != 16, dtype not bf16/fp16, head_dim not 128/256, Hq not a multiple of Hkv) and on
    /// any other non-OK status.
    public static func batchedSDPA2Pass(queries: MLXArray, keys: MLXArray, values: MLXArray, scale: Float,
                                        mask: MLXArray? = nil) -> MLXArray? {
        guard queries.ndim == 4, keys.ndim == 4, values.ndim == 4, let code = dtypeCode(queries.dtype) else { return nil }
        let (B, Hq, T, D) = (queries.dim(0), queries.dim(1), queries.dim(2), queries.dim(3))
        let (Hkv, N) = (keys.dim(1), keys.dim(2))
        guard values.dim(3) == D, Hkv > 0 else { return nil }
        guard let (qA, qP) = dense(queries), let (kA, kP) = dense(keys, as: queries.dtype),
              let (vA, vP) = dense(values, as: queries.dtype), let (out, outP) = output(queries.shape, queries.dtype)
        else { return nil }
        var maskP: UnsafeMutableRawPointer? = nil
        var maskA: MLXArray? = nil
        if let mask {
            // the kernel reads a dense [B, Hq, 16, N] mask in the attention dtype
            guard let (mA, mP) = dense(MLX.broadcast(mask.asType(queries.dtype), to: [B, Hq, T, N])) else { return nil }
            (maskA, maskP) = (mA, mP)
        }
        let bytes = dflash_verify_sdpa_workspace_bytes(Int32(B), Int32(Hq), Int32(Hkv), Int32(D), Int32(N))
        let (wsP, wsBytes) = DFlashWorkspace.shared.device(atLeast: bytes)
        let st = dflash_verify_sdpa(qP, kP, vP, nil, nil, maskP, outP, wsP, wsBytes,
                                    Int32(B), Int32(Hq), Int32(Hkv), Int32(T), Int32(D), Int32(N), 0, 0, 0,
                                    scale, code, Int32(DFLASH_KV_DENSE.rawValue), DFlashCUDAStream.current)
        withExtendedLifetime((qA, kA, vA, maskA)) {}
        return ok(st) ? out : nil
    }
}
