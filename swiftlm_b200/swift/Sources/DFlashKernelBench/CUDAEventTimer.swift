// CUDAEventTimer.swift — device-side timing for DFlashKernelBench.
//
// Replaces timeEval of Sources/DFlashKernelBench/main.swift:33-39 (wall clock around MLX.eval): a pair of
// CUDA events recorded on the stream the kernels run on, so that a sample is the device time of the
// call and not the host's launch and synchronisation overhead.  measure (:42-57), printResult and the byte
// counts of the GB/s lines stay as they are; only the body of timeEval changes:
//
//     private func timeEval(_ body: () -> MLXArray) -> Double { CUDAEventTimer.shared.seconds(body) }
//
// The CUDA runtime is reached through the C target's module (CDFlashCUDA links cudart); the four
// functions used here are declared below so that the bench needs no CUDA headers of its own.

import CDFlashCUDA
import DFlash
import MLX

@_silgen_name("cudaEventCreate") private func cudaEventCreate(_ event: UnsafeMutablePointer<OpaquePointer?>) -> Int32
@_silgen_name("cudaEventRecord") private func cudaEventRecord(_ event: OpaquePointer?, _ stream: UnsafeMutableRawPointer?) -> Int32
@_silgen_name("cudaEventSynchronize") private func cudaEventSynchronize(_ event: OpaquePointer?) -> Int32
@_silgen_name("cudaEventElapsedTime") private func cudaEventElapsedTime(_ ms: UnsafeMutablePointer<Float>, _ start: OpaquePointer?, _ end: OpaquePointer?) -> Int32

final class CUDAEventTimer {
    static let shared = CUDAEventTimer()
    private var start: OpaquePointer?
    private var stop: OpaquePointer?

    private init() {
        _ = cudaEventCreate(&start)
        _ = cudaEventCreate(&stop)
    }

    /// Device time in seconds of the work `body` enqueues (the DFlashKernels entry points launch eagerly on
    /// DFlashCUDAStream.current, so the kernels sit between the two events).
    func seconds(_ body: () -> MLXArray) -> Double {
        _ = cudaEventRecord(start, DFlashCUDAStream.current)
        let arr = body()
        _ = cudaEventRecord(stop, DFlashCUDAStream.current)
        _ = cudaEventSynchronize(stop)
        MLX.eval(arr)
        var ms: Float = 0
        _ = cudaEventElapsedTime(&ms, start, stop)
        // a bounded device-side wait that gave up, or data out of range, shows here and not as a trap
        let status = dflash_device_status(DFlashCUDAStream.current)
        if status != 0 { print("dflash_device_status: \(status) \(String(cString: dflash_last_error_string()))") }
        return Double(ms) * 1e-3
    }
}
