// Drop-in replacement for the reference's lib/cuda/cudacaller.dart (same class, same static method, same
// argument meaning), bound to libflutter_ml_b200.so through the generated fml_bindings.dart.
//
// Differences from the file it replaces (lib/cuda/cudacaller.dart:25-60 of the reference):
//   * the library keeps one context, so nothing is created or destroyed per call;
//   * the Dart doubles cross the boundary as one Float64List and are narrowed to float32 in C
//     (fml_upload_f64) instead of one element at a time in a Dart loop;
//   * every status is checked; a failure throws a StateError carrying fml_last_error.
// NOT executed by this repository's tests: no Dart SDK is available where they run.  The struct layouts it relies
// on are generated from include/fml.h and checked against the header on the CPU.
import 'dart:ffi';
import 'dart:typed_data';

import 'package:ffi/ffi.dart';

import 'fml_bindings.dart';

class CudaCaller {
  static const String libraryPath = 'cuda_lib/libflutter_ml_b200.so';
  static final FmlBindings fml = FmlBindings(DynamicLibrary.open(libraryPath));
  static Pointer<FmlCtx>? _ctx;

  /// The process-wide context (device 0, TF32 products), created on first use.
  static Pointer<FmlCtx> get context {
    final existing = _ctx;
    if (existing != null) return existing;
    final cfg = calloc<FmlConfig>();
    final out = calloc<Pointer<FmlCtx>>();
    try {
      cfg.ref
        ..device = 0
        ..precision = FmlPrecision.FML_PREC_TF32
        ..workspaceBytes = 0;
      _check(fml.fmlInit(cfg, out), nullptr);
      return _ctx = out.value;
    } finally {
      calloc.free(cfg);
      calloc.free(out);
    }
  }

  static void _check(int status, Pointer<FmlCtx> ctx) {
    if (status != FmlStatus.FML_OK) {
      throw StateError('libflutter_ml_b200: ${fml.fmlLastError(ctx).toDartString()} (status $status)');
    }
  }

  static Pointer<Float> _deviceFrom(List<double> values) {
    final ctx = context;
    final slot = calloc<Pointer<Float>>();
    final host = calloc<Double>(values.length);
    try {
      host.asTypedList(values.length).setAll(0, values is Float64List ? values : Float64List.fromList(values));
      _check(fml.fmlAlloc(ctx, values.length, slot), ctx);
      _check(fml.fmlUploadF64(ctx, slot.value, host, values.length), ctx);
      _check(fml.fmlSync(ctx), ctx); // the staging copy below is freed on return
      return slot.value;
    } finally {
      calloc.free(host);
      calloc.free(slot);
    }
  }

  /// C[m x n] = A[m x k] . B[k x n], row-major flat lists, as in the reference.
  static List<double> matmult(List<double> matA, List<double> matB, int m, int k, int n) {
    if (matA.length != m * k) throw ArgumentError('Matrix A has ${matA.length} elements, expected ${m * k}');
    if (matB.length != k * n) throw ArgumentError('Matrix B has ${matB.length} elements, expected ${k * n}');
    final ctx = context;
    final a = _deviceFrom(matA), b = _deviceFrom(matB);
    final cSlot = calloc<Pointer<Float>>();
    final desc = calloc<FmlGemmDesc>();
    final host = calloc<Double>(m * n);
    try {
      _check(fml.fmlAlloc(ctx, m * n, cSlot), ctx);
      desc.ref
        ..M = m
        ..N = n
        ..K = k
        ..lda = k
        ..ldb = n
        ..ldc = n
        ..A = a
        ..B = b
        ..C = cSlot.value
        ..alpha = 1.0
        ..batch1 = 1
        ..batch2 = 1
        ..precision = -1; // every other field stays zero (calloc): no bias, no activation, no row epilogue
      _check(fml.fmlGemm(ctx, desc), ctx);
      _check(fml.fmlDownloadF64(ctx, host, cSlot.value, m * n), ctx); // waits for the product
      return Float64List.fromList(host.asTypedList(m * n));
    } finally {
      fml.fmlFree(ctx, a);
      fml.fmlFree(ctx, b);
      if (cSlot.value != nullptr) fml.fmlFree(ctx, cSlot.value);
      calloc.free(cSlot);
      calloc.free(desc);
      calloc.free(host);
    }
  }

  /// The legacy symbol with host float buffers, exactly as the reference called it.
  static void multiplyMatrices(Pointer<Float> a, Pointer<Float> b, Pointer<Float> c, int m, int k, int n) =>
      fml.multiplyMatrices(a, b, c, m, k, n);
}
