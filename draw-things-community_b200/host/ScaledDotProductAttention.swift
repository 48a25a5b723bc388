// Swift binding of libdtattn.so with the call shape of the reference's operator.
//
// The reference builds attention as `ScaledDotProductAttention(scale:..., flags:...)(queries, keys, values)` and
// gets a `Model.IO` back (Flux1.swift:226-232, Qwen3_5.swift:193-197); a 4th positional input is the mask
// (Llama.swift:70-73) or the sinks (DeepSeek4.swift:488-493), and the variable-length form passes an array
// `([q, k, v, sequenceOffsets, sequenceOffsets])` (Qwen3_5VL.swift:431-435).  This class keeps those labels and
// those positional shapes on plain device views.
//
// What it is NOT: it is not the s4nnc `Model` subclass.  `Model.IO` is a symbolic graph value and the call sites
// go on with `.reshaped(...)` and `.add(dependencies:)`; a `DeviceView` is a concrete buffer.  Inside s4nnc the
// node's forward (where tensors and the CUDA stream are concrete) calls this class; the `Model` conformance, shape
// inference and parameter plumbing around it stay to be written there.  NOT COMPILED in this repository's build
// environment (no Swift toolchain).  `CDTAttn` is a module map over include/dtattn.h.
import CDTAttn

public struct GEMMFlag: OptionSet {
  public let rawValue: UInt32
  public init(rawValue: UInt32) { self.rawValue = rawValue }
  public static let Float16 = GEMMFlag(rawValue: 1)
  public static let Float32 = GEMMFlag(rawValue: 2)
  public static let Int8 = GEMMFlag(rawValue: 4)
}

/// A dense-innermost view of device memory: shape and element strides of any rank.  Attention tensors are
/// [B, S, H, D]; a mask is [B or 1, H or 1, Sq, Sk]; sinks are [1, 1, H, 1]; sequence offsets are [n + 1] Int32.
public struct DeviceView {
  public var pointer: UnsafeMutableRawPointer
  public var shape: [Int]
  public var strides: [Int]
  public var dtype: dt_dtype
  public init(pointer: UnsafeMutableRawPointer, shape: [Int], strides: [Int]? = nil, dtype: dt_dtype) {
    self.pointer = pointer
    self.shape = shape
    self.dtype = dtype
    if let s = strides {
      self.strides = s
    } else {  // contiguous
      var acc = 1
      var st = [Int](repeating: 1, count: shape.count)
      for i in stride(from: shape.count - 1, through: 0, by: -1) { st[i] = acc; acc *= shape[i] }
      self.strides = st
    }
  }
  var elementSize: Int { dtype == DT_F32 ? 4 : 2 }
  var abi4: dt_tensor4 {
    precondition(shape.count == 4 && (strides[3] == 1 || shape[3] == 1), "expect [B, S, H, D] with contiguous D")
    return dt_tensor4(ptr: pointer, stride_b: Int64(strides[0]), stride_s: Int64(strides[1]), stride_h: Int64(strides[2]))
  }
  /// `.reshaped(_:offset:strides:)` of the reference's views (Flux1.swift:236-243): same memory, new geometry.
  public func reshaped(_ shape: [Int], offset: [Int]? = nil, strides: [Int]? = nil) -> DeviceView {
    var p = pointer
    if let off = offset {
      precondition(off.count == self.strides.count)
      p = p + zip(off, self.strides).reduce(0) { $0 + $1.0 * $1.1 } * elementSize
    }
    return DeviceView(pointer: p, shape: shape, strides: strides, dtype: dtype)
  }
}

public final class ScaledDotProductAttention {
  /// Device memory for outputs and scratch comes from the host framework (the reference's graph executor owns the
  /// device allocator); the closure is called at most once per output and when the scratch has to grow.
  public typealias Allocator = (_ bytes: Int) -> UnsafeMutableRawPointer

  public let scale: Float
  public let isCausal: Bool
  public let hasAttentionMask: Bool
  public let flags: GEMMFlag
  public let multiHeadOutputProjectionFused: Bool
  public let hasAttentionSinks: Bool
  public let slidingWindow: Int
  public let isVariableLength: Bool
  public let maxSequenceLength: (query: Int, keyValue: Int)?
  public let name: String
  /// The unify-heads Dense of `multiHeadOutputProjectionFused: true`: [C, H*D] weight and [C] bias in the tensors'
  /// type.  The reference copies them into the node's `.weight` / `.bias` parameters (UNet.swift:865-874).
  public var weight: DeviceView?
  public var bias: DeviceView?
  /// CUDA stream the node runs on (the graph's stream), and the allocator; both may be changed between calls.
  public var stream: UnsafeMutableRawPointer?
  public var allocator: Allocator

  private var workspace: UnsafeMutableRawPointer?
  private var workspaceBytes = 0

  /// Labels as at the reference's call sites, including hasAttentionSinks / slidingWindow
  /// (DeepSeek4.swift:482-493) and isVariableLength / maxSequenceLength (Qwen3_5VL.swift:428-437).
  public init(
    scale: Float, isCausal: Bool = false, hasAttentionMask: Bool = false, flags: GEMMFlag = [],
    multiHeadOutputProjectionFused: Bool = false, hasAttentionSinks: Bool = false, slidingWindow: Int = 0,
    isVariableLength: Bool = false, maxSequenceLength: (query: Int, keyValue: Int)? = nil, name: String = "",
    stream: UnsafeMutableRawPointer? = nil, allocator: @escaping Allocator
  ) {
    precondition(!flags.contains(.Int8), "quantised attention is a Metal-only level (DeviceCapability.swift:132-146)")
    precondition(!(hasAttentionMask && hasAttentionSinks), "the 4th input is either the mask or the sinks")
    self.scale = scale
    self.isCausal = isCausal
    self.hasAttentionMask = hasAttentionMask
    self.flags = flags
    self.multiHeadOutputProjectionFused = multiHeadOutputProjectionFused
    self.hasAttentionSinks = hasAttentionSinks
    self.slidingWindow = slidingWindow
    self.isVariableLength = isVariableLength
    self.maxSequenceLength = maxSequenceLength
    self.name = name
    self.stream = stream
    self.allocator = allocator
  }

  /// op(queries, keys, values[, mask | sinks][, queryOffsets, keyValueOffsets]) -> output, the reference's
  /// positional order.  The output is [B, Sq, H, D], or [B, Sq, C] with the fused output projection.
  @discardableResult
  public func callAsFunction(_ queries: DeviceView, _ keys: DeviceView, _ values: DeviceView, _ extra: DeviceView...) -> DeviceView {
    return forward([queries, keys, values] + extra)
  }

  /// The array-input form (`([q, k, v, sequenceOffsets, sequenceOffsets])`, Qwen3_5VL.swift:431-435).
  @discardableResult
  public func callAsFunction(_ inputs: [DeviceView]) -> DeviceView {
    return forward(inputs)
  }

  private func ensureWorkspace(_ bytes: Int) {
    if bytes > workspaceBytes {
      workspace = allocator(bytes)  // the previous block goes back to the framework's allocator with the graph
      workspaceBytes = bytes
      check(dt_sdpa_workspace_init(workspace, bytes, stream), "dt_sdpa_workspace_init")
    }
  }

  private func check(_ status: Int32, _ what: String) {
    // the reference's operator traps on misuse (precondition / fatalError); so does this binding
    precondition(status == DT_OK.rawValue, "\(what)(\(name)): \(String(cString: dt_status_string(status)))")
  }

  private func forward(_ inputs: [DeviceView]) -> DeviceView {
    precondition(inputs.count >= 3, "queries, keys, values")
    let q = inputs[0], k = inputs[1], v = inputs[2]
    var rest = inputs.dropFirst(3)
    var p = dt_sdpa_params()
    p.B = Int32(q.shape[0]); p.Sq = Int32(q.shape[1]); p.Hq = Int32(q.shape[2]); p.D = Int32(q.shape[3])
    p.Sk = Int32(k.shape[1]); p.Hkv = Int32(k.shape[2])
    p.dtype = Int32(q.dtype.rawValue)
    p.scale = scale
    p.is_causal = isCausal ? 1 : 0
    p.flags = flags.contains(.Float16) ? UInt32(DT_FLAG_FP16_ACCUM_HINT) : 0
    p.q = q.abi4; p.k = k.abi4; p.v = v.abi4
    if hasAttentionMask {
      guard let m = rest.popFirst() else { preconditionFailure("hasAttentionMask: the mask is the 4th input") }
      precondition(m.shape.count == 4 && m.shape[2] == q.shape[1] && m.shape[3] == k.shape[1], "mask is [B|1, H|1, Sq, Sk]")
      p.mask = UnsafeRawPointer(m.pointer)
      p.mask_stride_b = m.shape[0] > 1 ? Int64(m.strides[0]) : 0
      p.mask_stride_h = m.shape[1] > 1 ? Int64(m.strides[1]) : 0
      p.mask_stride_q = Int64(m.strides[2])
    }
    if hasAttentionSinks {
      guard let s = rest.popFirst() else { preconditionFailure("hasAttentionSinks: the sinks are the 4th input") }
      precondition(s.shape.reduce(1, *) == q.shape[2], "one sink per query head ([1, 1, H, 1], DeepSeek4.swift:482-487)")
      p.sinks = UnsafeRawPointer(s.pointer)
    }
    p.sliding_window = Int32(slidingWindow)
    if isVariableLength {
      guard let oq = rest.popFirst(), let ok = rest.popFirst() else {
        preconditionFailure("isVariableLength: query and key/value sequence offsets follow the tensors")
      }
      p.seq_offsets_q = UnsafePointer<Int32>(OpaquePointer(oq.pointer))
      p.seq_offsets_k = UnsafePointer<Int32>(OpaquePointer(ok.pointer))
      p.n_seq = Int32(oq.shape[0] - 1)
      p.max_seq_q = Int32(maxSequenceLength?.query ?? q.shape[1])
      p.max_seq_k = Int32(maxSequenceLength?.keyValue ?? k.shape[1])
    }
    precondition(rest.isEmpty, "more inputs than the operator was built for")

    if multiHeadOutputProjectionFused {
      guard let w = weight else { preconditionFailure("multiHeadOutputProjectionFused: set .weight (and .bias) first") }
      let c = w.shape[0]
      let out = DeviceView(pointer: allocator(q.shape[0] * q.shape[1] * c * q.elementSize),
                           shape: [q.shape[0], q.shape[1], c], dtype: q.dtype)
      var proj = dt_out_proj()
      proj.weight = UnsafeRawPointer(w.pointer)
      proj.bias = bias.map { UnsafeRawPointer($0.pointer) }
      proj.C = Int32(c)
      proj.out = dt_tensor4(ptr: out.pointer, stride_b: Int64(out.strides[0]), stride_s: Int64(out.strides[1]), stride_h: Int64(c))
      p.o = p.q  // placeholder: the attention output stays in the workspace
      var bytes = 0
      check(dt_sdpa_projected_workspace_size(&p, &proj, &bytes), "dt_sdpa_projected_workspace_size")
      ensureWorkspace(bytes)
      check(dt_sdpa_forward_projected(&p, &proj, workspace, workspaceBytes, stream), "dt_sdpa_forward_projected")
      return out
    }
    let out = DeviceView(pointer: allocator(q.shape.reduce(1, *) * q.elementSize), shape: q.shape, dtype: q.dtype)
    p.o = out.abi4
    var bytes = 0
    check(dt_sdpa_workspace_size(&p, &bytes), "dt_sdpa_workspace_size")
    ensureWorkspace(bytes)
    check(dt_sdpa_forward(&p, workspace, workspaceBytes, stream), "dt_sdpa_forward")
    return out
  }

  /// One KV-cache step in one launch (Qwen3_5.swift:164-196): optional qNorm / kNorm, `Functional.cmul` with the
  /// rotary rows of the new tokens on the last `queries.shape[1]` queries and on the new keys, `moved(to:)` of the
  /// new keys and values into rows [cachedTokenLength, cachedTokenLength + T_new) of the caches, then this
  /// operator (isCausal) over cachedTokenLength + T_new rows.  keyCache / valueCache are views of the whole
  /// cache ([B, capacity, Hkv, D], Qwen3_5TextGeneration.swift:1639-1655); rotary is [B or 1, T_new, D].
  @discardableResult
  public func decodeStep(
    _ queries: DeviceView, keyCache: DeviceView, valueCache: DeviceView, newKeys: DeviceView, newValues: DeviceView,
    rotary: DeviceView?, cachedTokenLength: Int, qNormWeight: DeviceView? = nil, kNormWeight: DeviceView? = nil,
    normEpsilon: Float = 1e-6, kvPrefixStable: Bool = false
  ) -> DeviceView {
    precondition(isCausal && !hasAttentionMask && !isVariableLength && !multiHeadOutputProjectionFused)
    var s = dt_decode_step_params()
    let tNew = newKeys.shape[1]
    s.attn.B = Int32(queries.shape[0]); s.attn.Sq = Int32(queries.shape[1]); s.attn.Sk = Int32(cachedTokenLength + tNew)
    s.attn.Hq = Int32(queries.shape[2]); s.attn.Hkv = Int32(keyCache.shape[2]); s.attn.D = Int32(queries.shape[3])
    s.attn.dtype = Int32(queries.dtype.rawValue)
    s.attn.scale = scale
    s.attn.is_causal = 1
    s.attn.flags = (flags.contains(.Float16) ? UInt32(DT_FLAG_FP16_ACCUM_HINT) : 0) | (kvPrefixStable ? UInt32(DT_FLAG_KV_PREFIX_STABLE) : 0)
    s.attn.sliding_window = Int32(slidingWindow)
    let out = DeviceView(pointer: allocator(queries.shape.reduce(1, *) * queries.elementSize), shape: queries.shape, dtype: queries.dtype)
    s.attn.q = queries.abi4; s.attn.k = keyCache.abi4; s.attn.v = valueCache.abi4; s.attn.o = out.abi4
    s.k_new = newKeys.abi4; s.v_new = newValues.abi4; s.T_new = Int32(tNew)
    if let r = rotary {
      s.rotary = UnsafeRawPointer(r.pointer)
      s.rotary_stride_b = r.shape[0] > 1 ? Int64(r.strides[0]) : 0
      s.rotary_stride_s = Int64(r.strides[1])
    }
    s.q_norm_weight = qNormWeight.map { UnsafeRawPointer($0.pointer) }
    s.k_norm_weight = kNormWeight.map { UnsafeRawPointer($0.pointer) }
    s.norm_eps = normEpsilon
    var bytes = 0
    check(dt_sdpa_decode_step_workspace_size(&s, &bytes), "dt_sdpa_decode_step_workspace_size")
    ensureWorkspace(bytes)
    check(dt_sdpa_decode_step(&s, workspace, workspaceBytes, stream), "dt_sdpa_decode_step")
    return out
  }

  /// The nodes in front of the attention node as one pass (Flux1.swift:164-188, Wan.swift:86-98,
  /// Qwen3_5.swift:164-182): RMSNorm (per head row, or over all channels of a token), `Functional.cmul` with the
  /// rotary table and a constant factor, for queries and keys together.  Outputs may be row-offset views of a
  /// joint buffer, which also does the reference's concat of text and image tokens.
  public struct Prologue {
    public var normWeight: DeviceView?
    public var normPerToken = false
    public var epsilon: Float = 1e-6
    public var rotary: DeviceView?  // [B or 1, S, H or 1, D]
    public var postScale: Float = 1
    public init() {}
    func params(_ x: DeviceView, _ y: DeviceView) -> dt_qk_prologue_params {
      var p = dt_qk_prologue_params()
      p.B = Int32(x.shape[0]); p.S = Int32(x.shape[1]); p.H = Int32(x.shape[2]); p.D = Int32(x.shape[3])
      p.dtype = Int32(x.dtype.rawValue)
      p.x = x.abi4; p.y = y.abi4
      p.norm_weight = normWeight.map { UnsafeRawPointer($0.pointer) }
      p.norm_per_token = normPerToken ? 1 : 0
      p.eps = epsilon
      if let r = rotary {
        p.rotary = UnsafeRawPointer(r.pointer)
        p.rotary_stride_b = r.shape[0] > 1 ? Int64(r.strides[0]) : 0
        p.rotary_stride_s = Int64(r.strides[1])
        p.rotary_stride_h = r.shape[2] > 1 ? Int64(r.strides[2]) : 0
      }
      p.post_scale = postScale
      return p
    }
  }
  public static func qkPrologue(
    queries: DeviceView, into queriesOut: DeviceView, _ q: Prologue, keys: DeviceView? = nil, into keysOut: DeviceView? = nil,
    _ k: Prologue? = nil, stream: UnsafeMutableRawPointer?
  ) {
    var pq = q.params(queries, queriesOut)
    var status: Int32
    if let kx = keys, let ky = keysOut {
      var pk = (k ?? q).params(kx, ky)
      status = dt_qk_prologue(&pq, &pk, stream)
    } else {
      status = dt_qk_prologue(&pq, nil, stream)
    }
    precondition(status == DT_OK.rawValue, "dt_qk_prologue: \(String(cString: dt_status_string(status)))")
  }
}

/// SparseIndexedAttention(scale:isCausal:hasAttentionSinks:slidingWindow:) with the reference's input order
/// (DeepSeek4.swift:521-545): op(queries, rawKeys, rawValues, compressedKeys, compressedValues, selectedRows, sinks).
/// selectedRows is an Int32 view [queryLength, selectedRowCount]; compressedKeys / compressedValues may be empty
/// (the reference passes a [0] tensor when there are no compressed rows yet).
public final class SparseIndexedAttention {
  public let scale: Float
  public let isCausal: Bool
  public let hasAttentionSinks: Bool
  public let slidingWindow: Int
  public var stream: UnsafeMutableRawPointer?
  public var allocator: ScaledDotProductAttention.Allocator

  public init(
    scale: Float, isCausal: Bool = true, hasAttentionSinks: Bool = true, slidingWindow: Int = 0,
    stream: UnsafeMutableRawPointer? = nil, allocator: @escaping ScaledDotProductAttention.Allocator
  ) {
    self.scale = scale
    self.isCausal = isCausal
    self.hasAttentionSinks = hasAttentionSinks
    self.slidingWindow = slidingWindow
    self.stream = stream
    self.allocator = allocator
  }

  @discardableResult
  public func callAsFunction(
    _ queries: DeviceView, _ rawKeys: DeviceView, _ rawValues: DeviceView, _ compressedKeys: DeviceView,
    _ compressedValues: DeviceView, _ selectedRows: DeviceView, _ sinks: DeviceView? = nil
  ) -> DeviceView {
    precondition(hasAttentionSinks == (sinks != nil), "hasAttentionSinks and the inputs disagree")
    var p = dt_sparse_indexed_params()
    p.B = Int32(queries.shape[0]); p.Sq = Int32(queries.shape[1]); p.Hq = Int32(queries.shape[2]); p.D = Int32(queries.shape[3])
    p.Hkv = Int32(rawKeys.shape[2]); p.Sr = Int32(rawKeys.shape[1])
    let compressedRows = compressedKeys.shape.count == 4 ? compressedKeys.shape[1] : 0
    p.Sc = Int32(compressedRows)
    p.n_selected = Int32(selectedRows.shape[1])
    p.dtype = Int32(queries.dtype.rawValue)
    p.scale = scale
    p.is_causal = isCausal ? 1 : 0
    p.sliding_window = Int32(slidingWindow)
    let out = DeviceView(pointer: allocator(queries.shape.reduce(1, *) * queries.elementSize), shape: queries.shape, dtype: queries.dtype)
    p.q = queries.abi4; p.o = out.abi4; p.k_raw = rawKeys.abi4; p.v_raw = rawValues.abi4
    if compressedRows > 0 { p.k_comp = compressedKeys.abi4; p.v_comp = compressedValues.abi4 }
    p.selected = UnsafePointer<Int32>(OpaquePointer(selectedRows.pointer))
    p.selected_stride_b = 0
    p.selected_stride_q = Int64(selectedRows.strides[0])
    p.sinks = sinks.map { UnsafeRawPointer($0.pointer) }
    let status = dt_sparse_indexed_attention(&p, stream)
    precondition(status == DT_OK.rawValue, "dt_sparse_indexed_attention: \(String(cString: dt_status_string(status)))")
    return out
  }
}
