package lantern

import scala.util.continuations._
import org.scala_lang.virtualized.virtualize
import org.scala_lang.virtualized.SourceContext

import scala.virtualization.lms._
import scala.virtualization.lms.common._

/**
  * `BackendB200`: the GPU tensor backend that emits calls into liblantern_b200.so.
  *
  * It implements `trait Backend` (TensorDifferentiation.scala:137-379) the way `BackendCublas` / `BackendCudnn` do
  * (TensorDslCublas.scala:112-896, TensorDslCudnn.scala:142-1939): every method splices C text into the staged program
  * with `unchecked`.  The difference is what the text says.  The reference prints cuBLAS / cuDNN calls with their
  * descriptors, workspaces and one-element alpha/beta arrays, plus launches of kernels it also prints; this backend
  * prints exactly one call of an `ltb_*` entry point of include/lantern_b200.h per method, with the raw arena
  * pointers, the shapes and the scalars by value.  Results (loss, every gradient) follow the reference's CPU backend
  * (TensorDslCPU.scala); gradients ACCUMULATE into their destinations, as there.
  *
  * The trait extends `TensorDslCublas` only for its transfer operations (`toGPU`, `toCPU`, `moveToGPU`, ...,
  * TensorDslCublas.scala:37-107), which are written against the `GPUOps` nodes that `DslGenB200` maps onto the
  * library; `BackendB200` itself extends `Backend` directly, so that no method can fall through to cuBLAS unnoticed.
  *
  * Methods that no staged application on the CNN / RNN training path uses (the DeepSpeech operator set, and the ones
  * that take Scala closures, which the reference's GPU backends leave unimplemented too, TensorDslCublas.scala:164-168)
  * are `???`, as they are there.
  */
trait TensorDslB200 extends TensorDslCublas {

  // Arena mark / reset around a training step (TensorDslCublas.scala:18-25).  The library zeroes a block when it hands it
  // out again, so the reset itself is pointer arithmetic.
  override def getCudaMallocAddr(): Rep[Long] =
    unchecked[Long]("(long)ltb_mark()")
  override def resetCudaMallocAddr(addr: Rep[Long]) =
    unchecked[Unit]("LTB_CALL(ltb_reset((void*)", addr, "))")

  class BackendB200 protected() extends Backend {

    // ---- how a call is printed -------------------------------------------------------------------------------------
    // ltb("gemm", a, b, ...) prints  LTB_CALL(ltb_gemm(a, b, ...));  each Scala argument is one C argument.  An argument
    // may be a Rep, a Scala constant, a String of C text, or a Seq of those (printed back to back).
    private def flat(a: Any): Seq[Any] = a match {
      case s: Seq[_] => s.flatMap(flat)
      case b: Boolean => Seq(if (b) 1 else 0)
      case other => Seq(other)
    }
    private def commaSeparated(args: Seq[Any]): Seq[Any] =
      args.zipWithIndex.flatMap { case (a, i) => (if (i == 0) Seq() else Seq(", ")) ++ flat(a) }
    protected def ltb(fn: String, args: Any*): Rep[Unit] =
      unchecked[Unit]((Seq(s"LTB_CALL(ltb_$fn(") ++ commaSeparated(args) ++ Seq("))")): _*)

    // An int array argument (a broadcast shape, the extents of concat): a C++11 initializer list, alive until the call returns.
    private def ints(xs: Seq[Rep[Int]]): Seq[Any] =
      Seq("std::initializer_list<int>{") ++ commaSeparated(xs) ++ Seq("}.begin()")
    private def floatPtrs(ps: Seq[Any], const: Boolean): Seq[Any] =
      Seq(if (const) "std::initializer_list<const float*>{" else "std::initializer_list<float*>{") ++ commaSeparated(ps) ++ Seq("}.begin()")
    private val NULL = "NULL"
    private def gradOrNull(t: TensorR): Any = if (t.isInput) NULL else t.d.data          // a leaf has no gradient buffer to add into

    // Result buffers that the call overwrites completely skip the arena's zero fill.
    private def mallocUninit(n: Rep[Int]): Rep[Array[Float]] =
      unchecked[Array[Float]]("(float*)ltb_malloc_uninit((size_t)(", n, ") * sizeof(float))")
    private def mallocUninitInt(n: Rep[Int]): Rep[Array[Int]] =
      unchecked[Array[Int]]("(int*)ltb_malloc_uninit((size_t)(", n, ") * sizeof(int))")
    private def product(xs: Seq[Rep[Int]]): Rep[Int] = xs.foldLeft(unit(1)) { case (a, b) => a * b }

    // ---- lifetime, arena, initialisation (TensorDifferentiation.scala:139-179) ---------------------------------------
    // ltb_set_fusion(2): every device operation of a staged program goes through this library, so its one-call look-ahead
    // (batch norm or add joined by the in-place ReLU that follows, and the mirror image in backward) is safe; and in
    // reverse-mode code the gradient of a tensor is read by the backward code of its producer only, so the buffer that an
    // absorbed in-place ReLU gradient works on has no reader left (level 2: the mask is applied on load, not written back).
    // ltb_set_filter_cache(1): a staged program writes its filters only through the optimizer, transfer and fill entry
    // points, which is what the cache of per-tap filter forms relies on.
    override def setup(): Unit = {
      ltb("init", 0, "HEAP_SIZE")
      ltb("set_fusion", 2)
      ltb("set_filter_cache", 1)
    }
    override def cleanup(): Unit = ltb("shutdown")

    override def mallocArray[T: Manifest](length: Rep[Int]): Rep[Array[T]] = NewGPUArray[T](length)

    override def copyFloatArray(dest: Rep[Array[Float]], src: Rep[Array[Float]], length: Rep[Int]): Unit =
      ltb("d2d", dest, src, Seq("(size_t)(", length, ") * sizeof(float)"))

    override def arrayToTensor(array: Rep[Array[Float]], dims: Rep[Int]*): Tensor = new Tensor(array, dims)

    // Small constant tensors are built on the host and uploaded, as the cuBLAS backend does (TensorDslCublas.scala:133-134).
    override def makeTensor(dims: Seq[Rep[Int]], scalars: Float*): Tensor =
      BackendCPU().makeTensor(dims, scalars: _*).toGPU()

    override def fill(dims: Seq[Rep[Int]], value: Rep[Float]): Tensor = {
      val size = product(dims)
      val res = mallocUninit(size)
      ltb("fill", res, value, size)
      Tensor(res, dims: _*)
    }

    override def fillWithBias(dims: Seq[Rep[Int]], bias: Tensor, dim: Int): Tensor = {
      val res = mallocUninit(product(dims))
      ltb("fill_with_bias", res, bias.data, product(dims.take(dim)), dims(dim), product(dims.drop(dim + 1)))
      Tensor(res, dims: _*)
    }

    override def fillInPlace(x: Tensor, value: Rep[Float]): Unit = ltb("fill", x.data, value, x.scalarCount)

    // Drawn on the host from glibc rand() in element order and uploaded: the stream the CPU backend consumes
    // (TensorDslCPU.scala:101-110), which is what the reference's GPU backends do as well (TensorDslCublas.scala:154-155).
    override def randinit(dims: Seq[Int], scale: Float = 1.0f, seed: Option[Int] = None): Tensor = {
      val size = dims.product
      val res = mallocUninit(unit(size))
      ltb("randinit", res, size, scale, seed.getOrElse(-1))
      Tensor(res, dims.map(unit(_)): _*)
    }

    override def clipAt(x: Tensor, bound: Float) = ltb("clip", x.data, bound, x.scalarCount)

    // These take Scala closures; no C entry point can stand for them (also ??? in TensorDslCublas.scala:164-168).
    override def mutate(x: Tensor, delta: Rep[Int] => Rep[Float]): Unit = ???
    override def mapInPlace(x: Tensor, op: Rep[Float] => Rep[Float]): Unit = ???
    override def changeTo(x: Tensor, gen: Rep[Int] => Rep[Float]): Unit = ???
    override def map(x: Tensor, op: Rep[Float] => Rep[Float]): Tensor = ???
    override def fold(init: Rep[Float])(x: Tensor, op: (Rep[Float], Rep[Float]) => Rep[Float]): Rep[Float] = ???

    // ---- dot family (TensorDifferentiation.scala:186-219, TensorDslCPU.scala:135-225) -------------------------------------
    override def vectorVectorDot(x: Tensor, y: Tensor): Tensor = {
      val res = mallocUninit(1)
      ltb("vv_dot", x.data, y.data, res, x.shape(0))
      Tensor(res, 1)
    }

    override def matrixVectorDot(x: Tensor, y: Tensor): Tensor = {
      val res = mallocUninit(x.shape(0))
      ltb("mv_dot", x.data, y.data, res, x.shape(0), x.shape(1))
      Tensor(res, x.shape(0))
    }

    override def matrixMatrixDot(x: Tensor, y: Tensor): Tensor = {
      val res = mallocUninit(x.shape(0) * y.shape(1))
      ltb("mm_dot", x.data, y.data, res, x.shape(0), x.shape(1), y.shape(1))
      Tensor(res, x.shape(0), y.shape(1))
    }

    override def dot_grad(x: TensorR, y: TensorR, output: TensorR): Unit = {
      (x.x.rank, y.x.rank) match {
        case (1, 1) =>
          ltb("vv_dot_grad", gradOrNull(x), gradOrNull(y), x.x.data, y.x.data, output.d.data, x.x.shape(0))
        case (2, 1) =>
          if (!x.isInput) add_cartesian(x.d, y.x, output.d)
          if (!y.isInput) add_composition(y.d, x.x, output.d)
        case (2, 2) =>
          if (!x.isInput) add_dotTrans2(x.d, output.d, y.x)
          if (!y.isInput) add_dotTrans1(y.d, x.x, output.d)
      }
    }

    // x[i][j] += y[j] * output[i]
    override def add_cartesian(x: Tensor, y: Tensor, output: Tensor): Unit =
      ltb("add_cartesian", x.data, y.data, output.data, x.shape(0), x.shape(1))
    // x += y^T . output
    override def add_composition(x: Tensor, y: Tensor, output: Tensor): Unit =
      ltb("add_composition", x.data, y.data, output.data, y.shape(0), y.shape(1))
    // x[k][n] += y^T[k][m] . output[m][n]
    override def add_dotTrans1(x: Tensor, y: Tensor, output: Tensor): Unit =
      ltb("add_dot_trans1", x.data, y.data, output.data, y.shape(0), y.shape(1), output.shape(1))
    // x[m][k] += y[m][n] . output^T[n][k]
    override def add_dotTrans2(x: Tensor, y: Tensor, output: Tensor): Unit =
      ltb("add_dot_trans2", x.data, y.data, output.data, x.shape(0), x.shape(1), output.shape(1))

    // ---- broadcasting elementwise (TensorDifferentiation.scala:222-258, TensorDslCPU.scala:227-374) ---------------------
    private val ADD = 0; private val SUB = 1; private val MUL = 2; private val DIV = 3     // LTB_ADD .. LTB_DIV

    private def withScalar(op: Int, x: Tensor, y: Rep[Float]): Tensor = {
      val res = mallocUninit(x.scalarCount)
      ltb("ew_scalar", op, x.data, y, res, x.scalarCount)
      Tensor(res, x.shape: _*)
    }
    private def withTensor(op: Int, x: Tensor, y: Tensor): (Tensor, Dimensions, Dimensions) =
      Tensor.dimBroadcast(x.shape, y.shape) match {
        case Some((xShape, yShape, resShape)) =>
          val res = mallocUninit(resShape.scalarCount)
          ltb("ew_binary", op, x.data, ints(xShape.dims), y.data, ints(yShape.dims), res, resShape.dims.size)
          (Tensor(res, resShape.dims: _*), xShape, yShape)
        case _ => ???
      }
    private def withTensorGrad(op: Int, x: TensorR, y: TensorR, output: TensorR, xShape: Dimensions, yShape: Dimensions): Unit =
      ltb("ew_binary_grad", op, x.x.data, gradOrNull(x), ints(xShape.dims), y.x.data, gradOrNull(y), ints(yShape.dims),
          output.d.data, xShape.dims.size)
    private def inPlaceScalar(op: Int, x: Tensor, y: Rep[Float]): Unit =
      ltb("ew_inplace_scalar", op, x.data, y, x.scalarCount)
    // x = x (op) y where y is broadcast to x's shape, or reduced into it when y is the larger one
    private def inPlaceTensor(op: Int, x: Tensor, y: Tensor): Unit =
      Tensor.dimBroadcast(x.shape, y.shape) match {
        case Some((xShape, yShape, _)) => ltb("ew_inplace", op, x.data, ints(xShape.dims), y.data, ints(yShape.dims), xShape.dims.size)
        case _ => ???
      }

    override def +(x: Tensor, y: Rep[Float]): Tensor = withScalar(ADD, x, y)
    override def +(x: Tensor, y: Tensor): (Tensor, Dimensions, Dimensions) = withTensor(ADD, x, y)
    override def add_grad(x: TensorR, y: TensorR, output: TensorR, xShape: Dimensions, yShape: Dimensions): Unit =
      withTensorGrad(ADD, x, y, output, xShape, yShape)
    override def +=(x: Tensor, y: Rep[Float]): Unit = inPlaceScalar(ADD, x, y)
    override def +=(x: Tensor, y: Tensor): Unit = inPlaceTensor(ADD, x, y)

    override def -(x: Tensor, y: Rep[Float]): Tensor = withScalar(SUB, x, y)
    override def -(x: Tensor, y: Tensor): (Tensor, Dimensions, Dimensions) = withTensor(SUB, x, y)
    override def minus_grad(x: TensorR, y: TensorR, output: TensorR, xShape: Dimensions, yShape: Dimensions): Unit =
      withTensorGrad(SUB, x, y, output, xShape, yShape)
    override def -=(x: Tensor, y: Rep[Float]): Unit = inPlaceScalar(SUB, x, y)
    override def -=(x: Tensor, y: Tensor): Unit = inPlaceTensor(SUB, x, y)

    override def *(x: Tensor, y: Rep[Float]): Tensor = withScalar(MUL, x, y)
    override def *(x: Tensor, y: Tensor): (Tensor, Dimensions, Dimensions) = withTensor(MUL, x, y)
    override def mul_grad(x: TensorR, y: TensorR, output: TensorR, xShape: Dimensions, yShape: Dimensions): Unit =
      withTensorGrad(MUL, x, y, output, xShape, yShape)
    override def *=(x: Tensor, y: Rep[Float]): Unit = inPlaceScalar(MUL, x, y)
    override def *=(x: Tensor, y: Tensor): Unit = inPlaceTensor(MUL, x, y)

    override def /(x: Tensor, y: Rep[Float]): Tensor = withScalar(DIV, x, y)
    override def /(x: Tensor, y: Tensor): (Tensor, Dimensions, Dimensions) = withTensor(DIV, x, y)
    override def div_grad(x: TensorR, y: TensorR, output: TensorR, xShape: Dimensions, yShape: Dimensions): Unit =
      withTensorGrad(DIV, x, y, output, xShape, yShape)
    override def /=(x: Tensor, y: Rep[Float]): Unit = inPlaceScalar(DIV, x, y)
    override def /=(x: Tensor, y: Tensor): Unit = inPlaceTensor(DIV, x, y)

    // In place on `main`, which is returned (TensorDslCPU.scala:281-296).
    override def plusBias(main: Tensor, bias: Tensor): Tensor =
      Tensor.dimBroadcast(main.shape, bias.shape) match {
        case Some((mShape, bShape, _)) =>
          ltb("plus_bias", main.data, ints(mShape.dims), bias.data, ints(bShape.dims), mShape.dims.size)
          main
        case _ => ???
      }
    override def plusBias_grad(main: TensorR, bias: TensorR): Unit =
      if (!bias.isInput) Tensor.dimBroadcast(main.d.shape, bias.d.shape) match {
        case Some((mShape, bShape, _)) =>
          ltb("plus_bias_grad", bias.d.data, ints(bShape.dims), main.d.data, ints(mShape.dims), mShape.dims.size)
        case _ => ???
      }
    override def plusEqual(base: Tensor, adder: Tensor): Tensor = { inPlaceTensor(ADD, base, adder); base }
    override def plusEqual_grad(base: TensorR, adder: TensorR): Unit =
      if (!adder.isInput) inPlaceTensor(ADD, adder.d, base.d)

    // output = alpha * op(x) + beta * op(y); a tensor of rank other than 2 is treated as one row.
    override def geam(x: Tensor, transX: Boolean, alpha: Rep[Float], y: Tensor, transY: Boolean, beta: Rep[Float], output: Tensor): Unit = {
      val (rows, cols) = if (output.rank == 2) (output.shape(0), output.shape(1)) else (unit(1), output.scalarCount)
      ltb("geam", x.data, transX, alpha, y.data, transY, beta, output.data, rows, cols)
    }
    override def trans(x: Tensor): Tensor = {
      val res = mallocUninit(x.scalarCount)
      ltb("trans", x.data, res, x.shape(0), x.shape(1))
      Tensor(res, x.shape(1), x.shape(0))
    }
    override def trans_grad(x: TensorR, y: TensorR): Unit =
      ltb("trans_grad", x.d.data, y.d.data, x.x.shape(0), x.x.shape(1))

    // DeepSpeech only (DeepSpeech.scala:62, 133).
    override def permute(x: Tensor, dims: Int*): Tensor = ???
    override def permute_grad(x: TensorR, y: TensorR, dims: Int*): Unit = ???

    // ---- gemm (TensorDifferentiation.scala:279-280, TensorDslCPU.scala:379-472) ------------------------------------------
    override def gemm(x: Tensor, transX: Boolean, y: Tensor, transY: Boolean, alpha: Float): Tensor = {
      val m = if (transX) x.shape(1) else x.shape(0)
      val k = if (transX) x.shape(0) else x.shape(1)
      val n = if (transY) y.shape(0) else y.shape(1)
      val res = mallocUninit(m * n)
      ltb("gemm", x.data, transX, y.data, transY, alpha, res, m, n, k)
      Tensor(res, m, n)
    }
    override def gemm_grad(x: TensorR, transX: Boolean, y: TensorR, transY: Boolean, alpha: Float, output: TensorR): Unit = {
      val k = if (transX) x.x.shape(0) else x.x.shape(1)
      ltb("gemm_grad", x.x.data, gradOrNull(x), transX, y.x.data, gradOrNull(y), transY, alpha, output.d.data,
          output.x.shape(0), output.x.shape(1), k)
    }

    // ---- convolution (TensorDifferentiation.scala:292-296, TensorDslCPU.scala:484-692) -----------------------------------
    // pads of size 1 -> (p, p), 2 -> (p0, p1), 4 -> (p0, p2): TensorDslCPU.scala:533-534.
    private def padsOf(pads: Seq[Int]): (Int, Int) =
      if (pads.size == 1) (pads(0), pads(0)) else if (pads.size == 2) (pads(0), pads(1)) else (pads(0), pads(2))
    private def outSize(size: Rep[Int], kernel: Rep[Int], stride: Int, pad: Int): Rep[Int] = (size + 2 * pad - kernel) / stride + 1

    // No unfolded input crosses the boundary (the CPU backend hands its `finput` to backward, TensorDslCPU.scala:546-571) and
    // there is no per-site algorithm counter (TensorDslCudnn.scala:515-624): the library plans every call from its shapes.
    override def conv2D_batch(input: Tensor, kernel: Tensor, bias: Option[Tensor], strides: Seq[Int], pads: Seq[Int]): (Tensor, Option[Tensor], Int) = {
      val (ph, pw) = padsOf(pads)
      val ho = outSize(input.shape(2), kernel.shape(2), strides(0), ph)
      val wo = outSize(input.shape(3), kernel.shape(3), strides(1), pw)
      val res = mallocUninit(input.shape(0) * kernel.shape(0) * ho * wo)
      val biasData: Any = bias match { case Some(b) => b.data; case None => NULL }
      ltb("conv2d_fwd", input.data, kernel.data, biasData, res,
          input.shape(0), input.shape(1), input.shape(2), input.shape(3), kernel.shape(0), kernel.shape(2), kernel.shape(3),
          strides(0), strides(1), ph, pw)
      (Tensor(res, input.shape(0), kernel.shape(0), ho, wo), None, 0)
    }

    @virtualize
    override def conv2D_batch_grad(input: TensorR, finput: Option[TensorR], filter: TensorR, res: TensorR, bias: Option[TensorR] = None,
                                   padding: (Int, Int), strides: (Int, Int), dilations: (Int, Int), counter: Int): Unit = {
      assert(dilations._1 == 1 && dilations._2 == 1, "the library's convolution has dilation 1")
      val dbias: Any = bias match { case Some(b) => b.d.data; case None => NULL }
      ltb("conv2d_bwd", input.x.data, gradOrNull(input), filter.x.data, filter.d.data, dbias, res.d.data,
          input.x.shape(0), input.x.shape(1), input.x.shape(2), input.x.shape(3), filter.x.shape(0), filter.x.shape(2), filter.x.shape(3),
          strides._1, strides._2, padding._1, padding._2)
    }

    // ---- pooling (TensorDifferentiation.scala:298-302, TensorDslCPU.scala:848-1038) --------------------------------------
    // The saved indices are the CPU backend's: the first strict maximum, as a flat int32 index into the whole batch tensor.
    override def maxPool2D_batch(input: Tensor, kernel: Seq[Int], strides: Seq[Int], pads: Option[Seq[Int]]): (Tensor, Option[Rep[Array[Int]]]) = {
      val pad = pads match { case Some(p) => p(0); case None => 0 }
      val ho = outSize(input.shape(2), kernel(0), strides(0), pad)
      val wo = outSize(input.shape(3), kernel(1), strides(1), pad)
      val count = input.shape(0) * input.shape(1) * ho * wo
      val res = mallocUninit(count)
      val idx = mallocUninitInt(count)
      ltb("maxpool_fwd", input.data, res, idx, input.shape(0), input.shape(1), input.shape(2), input.shape(3),
          kernel(0), kernel(1), strides(0), strides(1), pad)
      (Tensor(res, input.shape(0), input.shape(1), ho, wo), Some(idx))
    }
    override def maxPool2D_batch_grad(input: TensorR, output: TensorR, sidx: Option[Rep[Array[Int]]], kernel: Seq[Int], strides: Seq[Int], pads: Seq[Int]): Unit =
      sidx match {
        case Some(idx) => ltb("maxpool_bwd", input.d.data, output.d.data, idx, Seq("(int64_t)", output.d.scalarCount))
        case None => ???
      }

    override def averagePool2D_batch(input: Tensor, kernel: Seq[Int], strides: Seq[Int], pads: Seq[Int]): Tensor = {
      assert(pads.forall(_ == 0), "average pooling takes no padding (TensorDslCPU.scala:1003-1005)")
      val ho = outSize(input.shape(2), kernel(0), strides(0), 0)
      val wo = outSize(input.shape(3), kernel(1), strides(1), 0)
      val res = mallocUninit(input.shape(0) * input.shape(1) * ho * wo)
      ltb("avgpool_fwd", input.data, res, input.shape(0), input.shape(1), input.shape(2), input.shape(3),
          kernel(0), kernel(1), strides(0), strides(1))
      Tensor(res, input.shape(0), input.shape(1), ho, wo)
    }
    override def averagePool2D_batch_grad(input: TensorR, output: TensorR, kernel: Seq[Int], strides: Seq[Int], pads: Seq[Int]): Unit =
      ltb("avgpool_bwd", input.d.data, output.d.data, input.x.shape(0), input.x.shape(1), input.x.shape(2), input.x.shape(3),
          kernel(0), kernel(1), strides(0), strides(1))

    // ---- batch norm (TensorDifferentiation.scala:304-306; TensorDslCPU.scala:1040-1056; TensorDslCudnn.scala:984-1131) ---
    // Spatial mode, epsilon 1e-5, running-average factor 0.1 (TensorDslCudnn.scala:1027); the saved statistics are the mean
    // and the inverse standard deviation, which backward takes back.
    override def batchNormInference(x: Tensor, scale: Tensor, bias: Tensor, runningMean: Tensor, runningVar: Tensor): Tensor = {
      val res = mallocUninit(x.scalarCount)
      ltb("bn_inference", x.data, res, scale.data, bias.data, runningMean.data, runningVar.data,
          x.shape(0), x.shape(1), x.shape(2) * x.shape(3), "1e-5f")
      Tensor(res, x.shape: _*)
    }
    override def batchNormTraining(x: Tensor, scale: Tensor, bias: Tensor, runningMean: Tensor, runningVar: Tensor): (Tensor, Option[Tensor], Option[Tensor], Int) = {
      val res = mallocUninit(x.scalarCount)
      val saveMean = mallocUninit(x.shape(1))
      val saveInvStd = mallocUninit(x.shape(1))
      ltb("bn_train_fwd", x.data, res, scale.data, bias.data, runningMean.data, runningVar.data, saveMean, saveInvStd,
          x.shape(0), x.shape(1), x.shape(2) * x.shape(3), "1e-5f", "0.1f")
      (Tensor(res, x.shape: _*), Some(Tensor(saveMean, x.shape(1))), Some(Tensor(saveInvStd, x.shape(1))), 0)
    }
    override def batchNorm_grad(input: TensorR, res: TensorR, scale: TensorR, bias: TensorR, saveMean: Option[Tensor], saveInvVariance: Option[Tensor], counterId: Int): Unit =
      (saveMean, saveInvVariance) match {
        case (Some(mean), Some(invStd)) =>
          ltb("bn_bwd", input.x.data, gradOrNull(input), res.d.data, scale.x.data, scale.d.data, bias.d.data, mean.data, invStd.data,
              input.x.shape(0), input.x.shape(1), input.x.shape(2) * input.x.shape(3))
        case _ => ???
      }

    // DeepSpeech only.
    override def batchNorm1DInference(x: Tensor, scale: Tensor, bias: Tensor, runningMean: Tensor, runningVar: Tensor): Tensor = ???
    override def batchNorm1DTraining(x: Tensor, scale: Tensor, bias: Tensor, runningMean: Tensor, runningVar: Tensor): (Tensor, Option[Tensor], Option[Tensor], Int) = ???
    override def batchNorm1D_grad(input: TensorR, res: TensorR, scale: TensorR, bias: TensorR, saveMean: Option[Tensor], saveInvVariance: Option[Tensor], counterId: Int): Unit = ???

    // ---- dropout (TensorDifferentiation.scala:312-313, TensorDslCPU.scala:1066-1088) ------------------------------------
    // The keep mask is drawn from glibc rand() on the host in element order, the CPU backend's stream, and uploaded.
    override def dropout(input: Tensor, prob: Float = 0.5f): (Tensor, Rep[Array[Float]], Rep[Int]) = {
      val res = mallocUninit(input.scalarCount)
      val mask = mallocUninit(input.scalarCount)
      ltb("dropout", input.data, res, mask, prob, Seq("(int64_t)", input.scalarCount))
      (Tensor(res, input.shape: _*), mask, input.scalarCount)
    }
    override def dropout_grad(input: TensorR, output: TensorR, prob: Float, helper: Rep[Array[Float]], size: Rep[Int]): Unit =
      ltb("dropout_grad", input.d.data, helper, output.d.data, Seq("(int64_t)", input.x.scalarCount))

    // DeepSpeech only.
    override def mask4D(input: Tensor, lengths: Rep[Array[Int]]): Tensor = ???

    // ---- activations (TensorDifferentiation.scala:319-335, TensorDslCPU.scala:710-781) -----------------------------------
    private val RELU = 0; private val TANH = 1; private val SIGMOID = 2; private val EXP = 3; private val LOG = 4
    private val SQRT = 5; private val SQUARE = 6                                              // LTB_RELU .. LTB_SQUARE

    private def unaryOp(op: Int, x: Tensor, inPlace: Boolean = false): Tensor = {
      val res = if (inPlace) x.data else mallocUninit(x.scalarCount)
      ltb("unary", op, x.data, res, Seq("(int64_t)", x.scalarCount))
      Tensor(res, x.shape: _*)
    }
    // In place (relu only): the caller's res is the input itself, the gradient buffer is masked where the value is not positive.
    private def unaryGrad(op: Int, input: TensorR, res: TensorR, inPlace: Boolean = false): Unit =
      ltb("unary_grad", op, input.x.data, input.d.data, res.x.data, res.d.data, Seq("(int64_t)", input.x.scalarCount), inPlace)

    override def relu(x: Tensor, inPlace: Boolean = false): Tensor = unaryOp(RELU, x, inPlace)
    override def tanh(x: Tensor): Tensor = unaryOp(TANH, x)
    override def sigmoid(x: Tensor): Tensor = unaryOp(SIGMOID, x)
    override def hardTanh(x: Tensor, min_val: Float = -1.0f, max_val: Float = 1.0f, inPlace: Boolean = false): Tensor = ???   // DeepSpeech only
    override def exp(x: Tensor): Tensor = unaryOp(EXP, x)
    override def log(x: Tensor): Tensor = unaryOp(LOG, x)
    override def sqrt(x: Tensor): Tensor = unaryOp(SQRT, x)
    override def square(x: Tensor): Tensor = unaryOp(SQUARE, x)

    override def relu_grad(input: TensorR, res: TensorR, inPlace: Boolean = false): Unit = unaryGrad(RELU, input, res, inPlace)
    override def tanh_grad(input: TensorR, res: TensorR): Unit = unaryGrad(TANH, input, res)
    override def sigmoid_grad(input: TensorR, res: TensorR): Unit = unaryGrad(SIGMOID, input, res)
    override def hardTanh_grad(input: TensorR, res: TensorR, min_val: Float = -1.0f, max_val: Float = 1.0f, inPlace: Boolean = false): Unit = ???
    override def exp_grad(input: TensorR, res: TensorR): Unit = unaryGrad(EXP, input, res)
    override def log_grad(input: TensorR, res: TensorR): Unit = unaryGrad(LOG, input, res)
    override def sqrt_grad(input: TensorR, res: TensorR): Unit = unaryGrad(SQRT, input, res)
    override def square_grad(input: TensorR, res: TensorR): Unit = unaryGrad(SQUARE, input, res)

    // ---- softmax family and the loss (TensorDifferentiation.scala:338-346, TensorDslCPU.scala:783-846, 1090-1110) ---------
    override def softmax(x: Tensor, dim: Int = 1): Tensor = {
      assert(x.rank == 2 && dim == 1, "softmax over the second of two dimensions (TensorDslCPU.scala:783-786)")
      val res = mallocUninit(x.scalarCount)
      ltb("softmax", x.data, res, x.shape(0), x.shape(1))
      Tensor(res, x.shape: _*)
    }
    override def logSoftmax(x: Tensor, dim: Int = 1): Tensor = {
      assert(x.rank == 2 && dim == 1, "logSoftmax over the second of two dimensions (TensorDslCPU.scala:805-808)")
      val res = mallocUninit(x.scalarCount)
      ltb("log_softmax", x.data, res, x.shape(0), x.shape(1))
      Tensor(res, x.shape: _*)
    }
    override def softmax_grad(input: TensorR, res: TensorR, dim: Int = 1): Unit =
      ltb("softmax_grad", input.d.data, res.x.data, res.d.data, res.x.shape(0), res.x.shape(1))
    override def logSoftmax_grad(input: TensorR, res: TensorR, dim: Int = 1): Unit =
      ltb("log_softmax_grad", input.d.data, res.x.data, res.d.data, res.x.shape(0), res.x.shape(1))

    override def nllLoss(x: Tensor, target: Rep[Array[Int]]): Tensor = {
      val res = mallocUninit(x.shape(0))
      ltb("nll", x.data, target, res, x.shape(0), x.shape(1))
      Tensor(res, x.shape(0))
    }
    override def nllLoss_grad(input: TensorR, res: TensorR, target: Rep[Array[Int]]): Unit =
      ltb("nll_grad", input.d.data, res.d.data, target, input.x.shape(0), input.x.shape(1))

    // DeepSpeech only.
    override def ctcLoss(prob: TensorR, inputLengths: Rep[Array[Int]], labels: Rep[Array[Int]], labelLengths: Rep[Array[Int]]): Tensor = ???

    // ---- reductions (TensorDifferentiation.scala:352-366, TensorDslCPU.scala:1115-1164) ----------------------------------
    override def sum(x: Tensor): Tensor = {
      val res = mallocUninit(1)
      ltb("sum", x.data, res, Seq("(int64_t)", x.scalarCount))
      Tensor(res, 1)
    }
    override def sum_grad(input: TensorR, res: TensorR): Unit =
      ltb("sum_grad", input.d.data, res.d.data, Seq("(int64_t)", input.x.scalarCount))
    override def mean(x: Tensor): Tensor = {
      val res = mallocUninit(1)
      ltb("mean", x.data, res, Seq("(int64_t)", x.scalarCount))
      Tensor(res, 1)
    }
    override def mean_grad(input: TensorR, res: TensorR): Unit =
      ltb("mean_grad", input.d.data, res.d.data, Seq("(int64_t)", input.x.scalarCount))

    override def sum(x: Tensor, dim: Int): Tensor = {
      val outer = product(x.shape.take(dim)); val inner = product(x.shape.drop(dim + 1))
      val res = mallocUninit(outer * inner)
      ltb("sum_dim", x.data, res, outer, x.shape(dim), inner)
      Tensor(res, (x.shape.take(dim) ++ x.shape.drop(dim + 1)): _*)
    }
    override def sum_grad(input: TensorR, output: TensorR, dim: Int): Unit = {
      val s = input.x.shape
      ltb("sum_dim_grad", input.d.data, output.d.data, product(s.take(dim)), s(dim), product(s.drop(dim + 1)))
    }

    // ---- concat (TensorDifferentiation.scala:369-370, TensorDslCPU.scala:1166-1212): any dimension, any number of inputs -
    override def concat(dim: Int, tensors: Seq[Tensor]): Tensor = {
      val first = tensors.head.shape
      val outer = product(first.take(dim)); val inner = product(first.drop(dim + 1))
      val extents = tensors.map(_.shape(dim))
      val total = extents.foldLeft(unit(0)) { case (a, b) => a + b }
      val res = mallocUninit(outer * total * inner)
      ltb("concat", res, floatPtrs(tensors.map(_.data), const = true), ints(extents), tensors.size, outer, inner)
      Tensor(res, (first.take(dim) ++ Seq(total) ++ first.drop(dim + 1)): _*)
    }
    override def concat_grad(dim: Int, tensorRs: Seq[TensorR], output: TensorR): Unit = {
      val first = tensorRs.head.x.shape
      ltb("concat_grad", floatPtrs(tensorRs.map(gradOrNull), const = false), output.d.data, ints(tensorRs.map(_.x.shape(dim))), tensorRs.size,
          product(first.take(dim)), product(first.drop(dim + 1)))
    }

    // DeepSpeech only.
    override def repeat0(in: Tensor, context: Int): Tensor = ???
    override def repeat0_grad(in: TensorR, out: TensorR, context: Int): Unit = ???

    // ---- optimizers (TensorDifferentiation.scala:377-378, TensorDslCPU.scala:1217-1246) ----------------------------------
    override def adagrad_update(tr: TensorR, t: Tensor, learning_rate: Float, gradClip: Float, descent: Boolean): Unit =
      ltb("adagrad_update", tr.x.data, tr.d.data, t.data, learning_rate, gradClip, descent, Seq("(int64_t)", tr.x.scalarCount))
    override def momentum_update(tr: TensorR, t: Tensor, learning_rate: Float, momentum: Float, gradClip: Float, nesterov: Boolean, descent: Boolean): Unit =
      ltb("momentum_update", tr.x.data, tr.d.data, t.data, learning_rate, momentum, gradClip, nesterov, descent, Seq("(int64_t)", tr.x.scalarCount))

    // The SGD module (NNModule.scala:265-287) issues geam(x, 1, d, -lr) and then fillInPlace(d, 0) per tensor; an Optim that
    // knows the library can emit the fused form instead: x -= lr * d; d = 0 in one pass (all-reduced first when the
    // communicator has more than one rank).
    def sgd_step(tr: TensorR, learning_rate: Float): Unit =
      ltb("allreduce_sgd_step", tr.x.data, tr.d.data, learning_rate, Seq("(int64_t)", tr.x.scalarCount))
  }

  object BackendB200 {
    def apply() = new BackendB200
  }

  // The default GPU backend (as TensorDslCudnn.scala:1946-1947 does for BackendCudnn).
  override def BackendGPU: Backend = BackendB200()
  backend = BackendGPU
}
