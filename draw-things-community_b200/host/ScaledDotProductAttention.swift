// Swift facade a maintainer of the reference would add to route its attention nodes to libdtattn.so.
// It keeps the initialiser labels the reference's call sites use (216 uses of `scale:`, 192 of `flags:`,
// 13 of `isCausal:`, 11 of `hasAttentionMask:`), so a model builder such as Flux1.swift:224-232 compiles
// unchanged against it.  NOT COMPILED in this repository's build environment (no Swift toolchain); it is
// shipped as the reference-side binding that INTEGRATION.md describes.  `CDTAttn` is a module map over
// include/dtattn.h.
import CDTAttn

public struct GEMMFlag: OptionSet {
  public let rawValue: UInt32
  public init(rawValue: UInt32) { self.rawValue = rawValue }
  public static let Float16 = GEMMFlag(rawValue: 1)
  public static let Float32 = GEMMFlag(rawValue: 2)
  public static let Int8 = GEMMFlag(rawValue: 4)
}

/// A [B, S, H, D] device view (element strides, D contiguous).
public struct DeviceView {
  public var pointer: UnsafeMutableRawPointer
  public var shape: (b: Int32, s: Int32, h: Int32, d: Int32)
  public var strides: (b: Int64, s: Int64, h: Int64)
  public var dtype: dt_dtype
  var abi: dt_tensor4 { dt_tensor4(ptr: pointer, stride_b: strides.b, stride_s: strides.s, stride_h: strides.h) }
}

public final class ScaledDotProductAttention {
  let scale: Float
  let isCausal: Bool
  let hasAttentionMask: Bool
  let flags: GEMMFlag
  let hasAttentionSinks: Bool
  let slidingWindow: Int
  let isVariableLength: Bool
  let maxSequenceLength: (query: Int, keyValue: Int)?

  /// Labels as at the reference's call sites, including hasAttentionSinks / slidingWindow
  /// (DeepSeek4.swift:482-493) and isVariableLength / maxSequenceLength (Qwen3_5VL.swift:428-437).
  public init(
    scale: Float, isCausal: Bool = false, hasAttentionMask: Bool = false, flags: GEMMFlag = [],
    multiHeadOutputProjectionFused: Bool = false, hasAttentionSinks: Bool = false, slidingWindow: Int = 0,
    isVariableLength: Bool = false, maxSequenceLength: (query: Int, keyValue: Int)? = nil, name: String = ""
  ) {
    self.hasAttentionSinks = hasAttentionSinks
    self.slidingWindow = slidingWindow
    self.isVariableLength = isVariableLength
    self.maxSequenceLength = maxSequenceLength
    precondition(!multiHeadOutputProjectionFused, "fused output projection is not provided by libdtattn")
    precondition(!flags.contains(.Int8), "quantised attention is a Metal-only level")
    self.scale = scale
    self.isCausal = isCausal
    self.hasAttentionMask = hasAttentionMask
    self.flags = flags
  }

  /// out = softmax(scale * Q K^T [+ mask]) V on `stream`; traps on misuse like the reference's operator.
  public func callAsFunction(
    _ queries: DeviceView, _ keys: DeviceView, _ values: DeviceView, mask: DeviceView? = nil,
    sinks: UnsafeRawPointer? = nil, sequenceOffsets: (query: UnsafePointer<Int32>, keyValue: UnsafePointer<Int32>, count: Int32)? = nil,
    out: DeviceView, workspace: UnsafeMutableRawPointer?, workspaceBytes: Int, stream: UnsafeMutableRawPointer?
  ) {
    precondition(hasAttentionMask == (mask != nil))
    var p = dt_sdpa_params()
    p.B = queries.shape.b; p.Sq = queries.shape.s; p.Sk = keys.shape.s
    p.Hq = queries.shape.h; p.Hkv = keys.shape.h; p.D = queries.shape.d
    p.dtype = Int32(queries.dtype.rawValue)
    p.scale = scale
    p.is_causal = isCausal ? 1 : 0
    p.flags = flags.contains(.Float16) ? UInt32(DT_FLAG_FP16_ACCUM_HINT) : 0
    p.q = queries.abi; p.k = keys.abi; p.v = values.abi; p.o = out.abi
    if let m = mask {
      p.mask = UnsafeRawPointer(m.pointer)
      p.mask_stride_b = m.shape.b > 1 ? m.strides.b : 0
      p.mask_stride_h = m.shape.s > 1 ? m.strides.s : 0
      p.mask_stride_q = m.strides.h
    }
    precondition(hasAttentionSinks == (sinks != nil) && isVariableLength == (sequenceOffsets != nil))
    p.sinks = sinks
    p.sliding_window = Int32(slidingWindow)
    if let o = sequenceOffsets {
      p.seq_offsets_q = o.query; p.seq_offsets_k = o.keyValue; p.n_seq = o.count
      p.max_seq_q = Int32(maxSequenceLength?.query ?? Int(p.Sq)); p.max_seq_k = Int32(maxSequenceLength?.keyValue ?? Int(p.Sk))
    }
    let status = dt_sdpa_forward(&p, workspace, workspaceBytes, stream)
    precondition(status == DT_OK.rawValue, String(cString: dt_status_string(status)))
  }
}
