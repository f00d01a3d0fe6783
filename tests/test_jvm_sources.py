"""The JVM-side sources (skainet_b200/jvm) cannot be compiled for real here (no JDK, no Kotlin). What can be checked is:
the JNI shim is valid C against a stand-in jni.h and only calls entry points include/*.h declares; every `external fun`
of CudaKernels.kt has its Java_..._CudaKernels_<name> twin in the shim with the same number of arguments; the
ServiceLoader files name classes the Kotlin sources define."""
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
JVM = os.path.join(ROOT, "skainet_b200", "jvm")
SHIM = os.path.join(JVM, "native", "skainet_cuda_jni.c")
KT = os.path.join(JVM, "src", "main", "kotlin", "sk", "ainet", "exec", "kernel", "cuda")


def split_args(s: str):
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch in "(<":
            depth += 1
        if ch in ")>":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur); cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur)
    return [a for a in out if a.strip()]


def shim_functions():
    text = open(SHIM).read()
    # expand the matvec macro instances
    fns = {}
    for m in re.finditer(r"JNI_FN\((\w+)\)\(JNIEnv\* env, jobject thiz(.*?)\)\s*\{", text, re.S):
        fns[m.group(1)] = len(split_args(m.group(2)))
    for m in re.finditer(r"^SKAINET_JNI_MATMUL\((\w+),", text, re.M):
        fns[m.group(1)] = 8
    fns.pop("jname", None)
    return fns


def test_shim_compiles_against_a_stand_in_jni_header(tmp_path):
    obj = str(tmp_path / "shim.o")
    r = subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-c", SHIM, "-I", os.path.join(ROOT, "tests", "stubs"),
                        "-I", os.path.join(ROOT, "include"), "-o", obj], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_shim_calls_only_declared_entry_points():
    declared = set()
    for h in ("skainet_cuda.h", "skainet_cuda_llama.h"):
        declared |= set(re.findall(r"\b(skainet_cuda_\w+)\s*\(", open(os.path.join(ROOT, "include", h)).read()))
    called = set(re.findall(r"\b(skainet_cuda_\w+)\s*\(", open(SHIM).read())) | set(re.findall(r"SKAINET_JNI_MATMUL\(\w+, (skainet_cuda_\w+)\)", open(SHIM).read()))
    assert called and called <= declared, called - declared


def test_every_external_fun_has_its_jni_twin_with_the_same_arity():
    kt = open(os.path.join(KT, "CudaKernels.kt")).read()
    ext = {m.group(1): len(split_args(m.group(2))) for m in re.finditer(r"external fun (\w+)\((.*?)\)\s*:", kt, re.S)}
    fns = shim_functions()
    assert ext and set(ext) == set(fns), (set(ext) ^ set(fns))
    for name, n in ext.items():
        assert fns[name] == n, (name, n, fns[name])
        assert "_" not in name        # JNI mangles underscores: the reference's rule


def test_service_files_name_defined_classes():
    sources = "".join(open(os.path.join(KT, f)).read() for f in os.listdir(KT))
    svc = os.path.join(JVM, "src", "main", "resources", "META-INF", "services")
    for f in ("sk.ainet.backend.api.kernel.KernelProvider", "sk.ainet.backend.api.kernel.ViewKernelPack"):
        cls = open(os.path.join(svc, f)).read().strip()
        assert cls.startswith("sk.ainet.exec.kernel.cuda.")
        assert re.search(r"public class %s\b" % cls.rsplit(".", 1)[1], sources), cls
