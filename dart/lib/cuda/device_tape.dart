// Runs an existing flutter_ml autograd graph on the GPU: walks the Node list of a loss tensor
// (Node.inputs / opName / extraParams, lib/autogradEngine/tensor.dart:5-19), mirrors every tensor in device memory
// and hands the whole list to fml_tape_run, one FFI call per sweep, in place of Tensor.backward's closure loop
// (tensor.dart:43-75).  The graph is built once by the unmodified layer code (forward on the CPU engine with the
// first sample); afterwards `forward()` / `backward()` re-run it on the device for new leaf values.
//
// NOT executed by this repository's tests (no Dart SDK where they run).  The same walker in Python
// (flutter_ml_b200/tape.py) drives the identical fml_op records through the identical entry point and is tested
// against the CPU oracle; the struct layout comes from the generated fml_bindings.dart.
import 'dart:ffi';
import 'dart:typed_data';

import 'package:ffi/ffi.dart';

import '../autogradEngine/tensor.dart';
import 'cudacaller.dart';
import 'fml_bindings.dart';

class _Mirror {
  final int rows, cols;
  Pointer<Float> value = nullptr, grad = nullptr;
  _Mirror(this.rows, this.cols);
  int get count => rows * cols;
}

class DeviceTape {
  final FmlBindings fml = CudaCaller.fml;
  final Pointer<FmlCtx> ctx = CudaCaller.context;
  final List<Node> _topo = [];
  final Map<Node, Tensor> _outputOf = {};
  final Map<Tensor, _Mirror> _mirrors = {};
  final List<Tensor> leaves = [];
  final List<Pointer<NativeType>> _owned = [];
  late final Pointer<FmlOp> _ops;

  /// Builds the device tape of `loss` (a tensor produced by the reference's ops).
  DeviceTape(Tensor loss) {
    _sort(loss);
    for (final node in _topo) {
      for (final t in node.inputs) {
        _mirror(t);
      }
      _mirror(_outputOf[node]!);
    }
    _ops = calloc<FmlOp>(_topo.length);
    for (var i = 0; i < _topo.length; i++) {
      _fill(_ops[i], _topo[i]);
    }
    uploadLeaves();
  }

  // Same order as Tensor.backward builds it (tensor.dart:54-66), remembering which tensor each node produced.
  void _sort(Tensor root) {
    final visited = <Node>{};
    void visit(Tensor t) {
      final n = t.creator;
      if (n == null || !visited.add(n)) return;
      _outputOf[n] = t;
      for (final input in n.inputs) {
        visit(input);
      }
      _topo.add(n);
    }
    visit(root);
  }

  static List<int> _shape(Tensor t) {
    final v = t.value;
    if (v is double) return [1, 1];
    if (v is List<List<double>>) return [v.length, v.isEmpty ? 0 : v[0].length];
    return [1, (v as List<double>).length];
  }

  _Mirror _mirror(Tensor t) => _mirrors.putIfAbsent(t, () {
        final s = _shape(t);
        final m = _Mirror(s[0], s[1]);
        final slot = calloc<Pointer<Float>>();
        _check(fml.fmlAlloc(ctx, m.count, slot));
        m.value = slot.value;
        _check(fml.fmlAlloc(ctx, m.count, slot));
        m.grad = slot.value;
        _check(fml.fmlZero(ctx, m.grad, m.count));
        calloc.free(slot);
        if (t.creator == null) leaves.add(t);
        return m;
      });

  void _fill(FmlOp op, Node node) {
    final kind = using((arena) => fml.fmlTapeKind(node.opName.toNativeUtf8(allocator: arena)));
    if (kind == 0) throw UnsupportedError('op "${node.opName}" has no device rule');
    final out = _mirrors[_outputOf[node]]!;
    final ins = node.inputs.map((t) => _mirrors[t]!).toList();
    op
      ..kind = kind
      ..rows = out.rows
      ..cols = out.cols
      ..out = out.value
      ..gout = out.grad
      ..precision = -1
      ..s = ((node.extraParams['s'] ?? node.extraParams['alpha'] ?? node.extraParams['epsilon'] ?? 0.0) as num).toDouble();
    if (kind == FmlOpKind.FML_OP_CONCAT) {
      final parts = calloc<Pointer<Float>>(ins.length), gparts = calloc<Pointer<Float>>(ins.length);
      final cols = calloc<Int32>(ins.length);
      for (var i = 0; i < ins.length; i++) {
        parts[i] = ins[i].value;
        gparts[i] = ins[i].grad;
        cols[i] = ins[i].cols;
      }
      _owned.addAll([parts, gparts, cols]);
      op
        ..parts = parts
        ..gparts = gparts
        ..partCols = cols
        ..nParts = ins.length;
      return;
    }
    for (var i = 0; i < ins.length && i < 3; i++) {
      op.inp[i] = ins[i].value;
      op.gin[i] = ins[i].grad;
    }
    switch (kind) {
      case FmlOpKind.FML_OP_MATMUL: // out[r x c] = in0[r x inner] . in1[inner x c]
      case FmlOpKind.FML_OP_MATVECMUL: // out[c] = in0[c x inner] . in1[inner]
        op.inner = ins[0].cols;
      case FmlOpKind.FML_OP_MSE:
      case FmlOpKind.FML_OP_SUM:
        op.inner = ins[0].count;
      case FmlOpKind.FML_OP_LAYER_NORM: // x-hat and 1/sigma are kept between the sweeps
        final slot = calloc<Pointer<Float>>();
        _check(fml.fmlAlloc(ctx, out.count, slot));
        op.aux[0] = slot.value;
        _check(fml.fmlAlloc(ctx, out.rows, slot));
        op.aux[1] = slot.value;
        calloc.free(slot);
      case FmlOpKind.FML_OP_CONV2D:
        final same = node.extraParams['padding'] == 'same';
        op
          ..inner = ins[1].rows
          ..iparam = ins[1].cols
          ..s = same ? ((ins[1].rows - 1) ~/ 2).toDouble() : 0.0;
    }
  }

  static Float64List _flatten(Tensor t) {
    final v = t.value;
    if (v is double) return Float64List.fromList([v]);
    if (v is List<List<double>>) return Float64List.fromList([for (final row in v) ...row]);
    return Float64List.fromList(v as List<double>);
  }

  /// Copies the current CPU values of every leaf (inputs, targets, parameters) to the device.
  void uploadLeaves() {
    for (final t in leaves) {
      final m = _mirrors[t]!;
      final flat = _flatten(t);
      final host = calloc<Double>(flat.length);
      host.asTypedList(flat.length).setAll(0, flat);
      _check(fml.fmlUploadF64(ctx, m.value, host, flat.length));
      _check(fml.fmlSync(ctx));
      calloc.free(host);
    }
  }

  void forward() => _check(fml.fmlTapeRun(ctx, _ops, _topo.length, FmlTapeDirection.FML_TAPE_FORWARD));

  /// Zeroes the gradients of intermediate tensors (every reference forward pass starts them at zero,
  /// tensor.dart:26-41), seeds the loss with 1 (tensor.dart:70) and runs every gradient rule last to first;
  /// leaf gradients accumulate until `zeroLeafGrads`, as Optimizer.zeroGrad expects (optimizers.dart:62-66).
  void backward() {
    for (final node in _topo) {
      final m = _mirrors[_outputOf[node]]!;
      _check(fml.fmlZero(ctx, m.grad, m.count));
    }
    _check(fml.fmlTapeRun(ctx, _ops, _topo.length, FmlTapeDirection.FML_TAPE_BACKWARD));
  }

  void zeroLeafGrads() {
    for (final t in leaves) {
      final m = _mirrors[t]!;
      _check(fml.fmlZero(ctx, m.grad, m.count));
    }
  }

  /// Device value (or gradient) of `t` as a flat row-major list of doubles.
  Float64List download(Tensor t, {bool grad = false}) {
    final m = _mirrors[t]!;
    final host = calloc<Double>(m.count);
    try {
      _check(fml.fmlDownloadF64(ctx, host, grad ? m.grad : m.value, m.count));
      return Float64List.fromList(host.asTypedList(m.count));
    } finally {
      calloc.free(host);
    }
  }

  void dispose() {
    for (final m in _mirrors.values) {
      fml.fmlFree(ctx, m.value);
      fml.fmlFree(ctx, m.grad);
    }
    for (var i = 0; i < _topo.length; i++) {
      for (var j = 0; j < 2; j++) {
        if (_ops[i].aux[j] != nullptr) fml.fmlFree(ctx, _ops[i].aux[j]);
      }
    }
    for (final p in _owned) {
      calloc.free(p);
    }
    calloc.free(_ops);
  }

  void _check(int status) {
    if (status != FmlStatus.FML_OK) {
      throw StateError('libflutter_ml_b200: ${fml.fmlLastError(ctx).toDartString()} (status $status)');
    }
  }
}
