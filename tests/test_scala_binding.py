"""The Scala side of the boundary (integration/scala) against the C header.

No JVM is needed: the Scala sources are read as text.  `BackendB200` prints every call through one helper,
`ltb("name", arg, arg, ...)`, one Scala argument per C argument, so the binding can be checked mechanically: every name
must be declared in include/lantern_b200.h with exactly that many parameters, and every `Backend` method that the
training path needs must be implemented (not left as `???`)."""
import os
import re

from lantern_b200 import parse_header

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCALA = os.path.join(ROOT, "integration", "scala")

# trait Backend methods (src/main/scala/lantern/TensorDifferentiation.scala:137-379) on the CNN / RNN training path
IN_SCOPE = """setup cleanup mallocArray copyFloatArray arrayToTensor makeTensor fill fillWithBias fillInPlace randinit clipAt
vectorVectorDot matrixVectorDot matrixMatrixDot dot_grad add_cartesian add_composition add_dotTrans1 add_dotTrans2
+ - * / += -= *= /= add_grad minus_grad mul_grad div_grad plusBias plusBias_grad plusEqual plusEqual_grad geam trans trans_grad
gemm gemm_grad conv2D_batch conv2D_batch_grad maxPool2D_batch maxPool2D_batch_grad averagePool2D_batch averagePool2D_batch_grad
batchNormInference batchNormTraining batchNorm_grad dropout dropout_grad relu tanh sigmoid exp log sqrt square
relu_grad tanh_grad sigmoid_grad exp_grad log_grad sqrt_grad square_grad softmax logSoftmax softmax_grad logSoftmax_grad
nllLoss nllLoss_grad sum sum_grad mean mean_grad concat concat_grad adagrad_update momentum_update""".split()
# ... and the ones only the DeepSpeech application or closure-taking callers need: present, but unimplemented as in the reference
OUT_OF_SCOPE = """mutate mapInPlace changeTo map fold permute permute_grad batchNorm1DInference batchNorm1DTraining batchNorm1D_grad
mask4D hardTanh hardTanh_grad ctcLoss repeat0 repeat0_grad""".split()


def _read(name):
    return open(os.path.join(SCALA, name)).read()


def _strip_comments(text):
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def _split_args(text, start):
    """Top-level arguments of the call whose opening parenthesis is at text[start]; returns (args, end index)."""
    depth, i, cur, args, in_str = 0, start, "", [], False
    while i < len(text):
        c = text[i]
        if in_str:
            cur += c
            if c == "\\":
                cur += text[i + 1]; i += 1
            elif c == '"':
                in_str = False
        elif c == '"':
            in_str = True; cur += c
        elif c in "([{":
            depth += 1
            if depth > 1:
                cur += c
        elif c in ")]}":
            depth -= 1
            if depth == 0:
                if cur.strip():
                    args.append(cur.strip())
                return args, i
            cur += c
        elif c == "," and depth == 1:
            args.append(cur.strip()); cur = ""
        else:
            cur += c
        i += 1
    raise ValueError("unbalanced call")


def _calls(text):
    """[(entry point name, number of C arguments)] of every ltb("name", ...) call."""
    out = []
    for m in re.finditer(r'\bltb\(\s*"(\w+)"', text):
        args, _ = _split_args(text, m.start() + 3)
        out.append((m.group(1), len(args) - 1))
    return out


def test_every_emitted_call_names_a_declared_entry_point_with_its_arity():
    decls = parse_header()
    text = _strip_comments(_read("TensorDslB200.scala"))
    calls = _calls(text)
    assert len(calls) >= 55, len(calls)
    for name, n in calls:
        assert name in decls, "BackendB200 emits ltb_%s, which include/lantern_b200.h does not declare" % name
        want = len(decls[name][1])
        assert n == want, "ltb_%s: BackendB200 passes %d arguments, the header declares %d" % (name, n, want)
    # calls printed as raw text (the arena's mark / reset, the uninitialised malloc, the generator's copies)
    raw = set(re.findall(r"\bltb_([a-z0-9_]*[a-z0-9])\b", text + _strip_comments(_read("DslGenB200.scala")))) - {""}   # names ending in _ are the macro's locals
    raw = {n for n in raw if not n.startswith("$")}
    assert {"mark", "reset", "malloc_uninit", "malloc", "h2d", "d2h", "d2d", "last_error"} <= raw
    for name in raw:
        assert name in decls, "ltb_%s is not declared in the header" % name


def test_every_backend_method_on_the_training_path_is_implemented():
    text = _strip_comments(_read("TensorDslB200.scala"))
    body = text[text.index("class BackendB200"):]
    for name in IN_SCOPE + OUT_OF_SCOPE:
        defs = re.findall(r"override\s+def\s+%s\s*[\[\(:=]([^\n]*)" % re.escape(name), body)
        assert defs, "BackendB200 does not override Backend.%s" % name
        stubbed = [d for d in defs if d.rstrip().endswith("= ???")]
        if name in IN_SCOPE:
            assert not stubbed, "Backend.%s is on the training path but left as ???" % name
        else:
            assert len(stubbed) == len(defs), "Backend.%s is declared out of scope but has a body" % name
    # both overloads of the binary operators and of sum / sum_grad exist
    for op in ("+", "-", "*", "/"):
        assert len(re.findall(r"override\s+def\s+%s\(x: Tensor, y: " % re.escape(op), body)) == 2
    assert len(re.findall(r"override\s+def\s+sum\(", body)) == 2 and len(re.findall(r"override\s+def\s+sum_grad\(", body)) == 2
    assert "override def BackendGPU: Backend = BackendB200()" in text


def test_generator_and_driver_replace_the_cudnn_ones():
    gen, drv = _strip_comments(_read("DslGenB200.scala")), _strip_comments(_read("LanternDriverB200.scala"))
    assert "trait DslGenB200 extends DslGenBase with CudaGenGPUOps" in gen and '"\\"lantern_b200.h\\""' in gen
    assert "LTB_CALL" in gen and "getCudaMallocArenaString" in gen and "override def cudaMemcpy" in gen
    assert re.search(r"abstract class LanternDriverB200\[A: Manifest, B: Manifest\] extends DslDriverB200\[A, B\]\s+with LanternDriver\[A, B\] with TensorDslB200", drv)
    assert "-llantern_b200" in drv and "cublas" not in drv and "cudnn" not in drv
