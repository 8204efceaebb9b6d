"""The JNI binders against a mock JVM: function tables with the JNI
specification's slot numbers, built with ctypes.  Checks JNI_OnLoad's field-id
lookup and the jcuda.Pointer -> device address unwrapping
(nativePointer + byteOffset, null object -> null)."""
import ctypes as C

import pytest

FIND_CLASS, GET_FIELD_ID, GET_LONG_FIELD, JVM_GET_ENV = 6, 94, 101, 6


class MockJVM:
    def __init__(self, fail_class=None):
        self.objects = {}      # handle -> {"nativePointer": .., "byteOffset": ..}
        self.classes = {}
        self.fields = {}
        self.lookups = []
        self.fail_class = fail_class

        @C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_char_p)
        def find_class(env, name):
            name = name.decode()
            self.lookups.append(("class", name))
            if name == self.fail_class:
                return None
            return self.classes.setdefault(name, 0x1000 + len(self.classes))

        @C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p, C.c_char_p)
        def get_field_id(env, cls, name, sig):
            self.lookups.append(("field", name.decode(), sig.decode()))
            return self.fields.setdefault(name.decode(), 0x2000 + len(self.fields))

        @C.CFUNCTYPE(C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p)
        def get_long_field(env, obj, fid):
            name = {v: k for k, v in self.fields.items()}[fid]
            return self.objects[obj][name]

        self._keep = (find_class, get_field_id, get_long_field)
        table = (C.c_void_p * 232)()
        table[FIND_CLASS] = C.cast(find_class, C.c_void_p)
        table[GET_FIELD_ID] = C.cast(get_field_id, C.c_void_p)
        table[GET_LONG_FIELD] = C.cast(get_long_field, C.c_void_p)
        self.table = table
        self.env = C.pointer(C.cast(table, C.c_void_p))  # JNIEnv* : pointer to pointer to table

        @C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_void_p), C.c_int)
        def get_env(vm, penv, version):
            penv[0] = C.cast(self.env, C.c_void_p)
            return 0

        self._keep += (get_env,)
        vtable = (C.c_void_p * 8)()
        vtable[JVM_GET_ENV] = C.cast(get_env, C.c_void_p)
        self.vtable = vtable
        self.vm = C.pointer(C.cast(vtable, C.c_void_p))

    def pointer(self, native, offset):
        h = 0x9000 + 16 * len(self.objects)
        self.objects[h] = {"nativePointer": native, "byteOffset": offset}
        return h


@pytest.fixture(scope="module")
def lib():
    from bidmach_b200 import _lib
    l = _lib.load()
    l.bidmach_jni_device_address.restype = C.c_void_p
    l.bidmach_jni_device_address.argtypes = [C.c_void_p, C.c_void_p]
    return l


def test_onload_caches_the_two_jcuda_fields(lib):
    jvm = MockJVM()
    assert lib.JNI_OnLoad(C.cast(jvm.vm, C.c_void_p), None) == 0x00010004
    assert ("class", "jcuda/NativePointerObject") in jvm.lookups
    assert ("class", "jcuda/Pointer") in jvm.lookups
    assert ("field", "nativePointer", "J") in jvm.lookups
    assert ("field", "byteOffset", "J") in jvm.lookups


def test_onload_fails_cleanly_without_jcuda(lib):
    jvm = MockJVM(fail_class="jcuda/Pointer")
    assert lib.JNI_OnLoad(C.cast(jvm.vm, C.c_void_p), None) == -1


def test_pointer_unwrap_is_native_pointer_plus_byte_offset(lib):
    jvm = MockJVM()
    assert lib.JNI_OnLoad(C.cast(jvm.vm, C.c_void_p), None) == 0x00010004
    env = C.cast(jvm.env, C.c_void_p)
    p = jvm.pointer(0x7F00_0000_1000, 0x240)
    assert lib.bidmach_jni_device_address(env, p) == 0x7F00_0000_1240
    assert lib.bidmach_jni_device_address(env, jvm.pointer(0x1000, 0)) == 0x1000
    assert lib.bidmach_jni_device_address(env, None) is None


def test_binders_forward_to_the_launchers(lib, capfd):
    """Zero columns and an unsupported shape return before any CUDA call, so the
    argument plumbing can be exercised on a machine without a GPU."""
    jvm = MockJVM()
    assert lib.JNI_OnLoad(C.cast(jvm.vm, C.c_void_p), None) == 0x00010004
    env = C.cast(jvm.env, C.c_void_p)
    ptrs = [jvm.pointer(0x10000 * (k + 1), 0) for k in range(6)]
    f = lib.Java_edu_berkeley_bid_CUMACH_word2vecPos
    assert f(env, None, 100, 10, 4, *ptrs[:5], 0.1, 0.5) == 1       # skip 4 is unsupported
    assert f(env, None, 2000, 10, 5, *ptrs[:5], 0.1, 0.5) == 1      # too many rows
    g = lib.Java_edu_berkeley_bid_CUMACH_word2vecNeg
    assert g(env, None, 100, 10, 3, 3, *ptrs[:4], 0.1, 0.5) == 1
    h = lib.Java_edu_berkeley_bid_CUMACH_word2vecEvalNeg
    assert h(env, None, 100, 10, 7, 7, *ptrs[:5]) == 1
    k = lib.Java_edu_berkeley_bid_CUMACH_word2vecNegFilt
    assert k(env, None, 100, 10, 50, 2, 2, *ptrs[:4], 0.1, 0.5) == 1
    e = lib.Java_edu_berkeley_bid_CUMACH_word2vecEvalPos
    assert e(env, None, 100, 10, 9, *ptrs[:6]) == 1


def test_slice_and_exchange_binders_check_their_arguments(lib, capfd):
    """The binders of the slice launchers and of the exchange: refusals that come back before any
    CUDA or NCCL call."""
    jvm = MockJVM()
    assert lib.JNI_OnLoad(C.cast(jvm.vm, C.c_void_p), None) == 0x00010004
    env = C.cast(jvm.env, C.c_void_p)
    ptrs = [jvm.pointer(0x10000 * (k + 1), 0) for k in range(6)]
    f = lib.Java_edu_berkeley_bid_CUMACH_word2vecPosSlice
    assert f(env, None, 100, 10, 5, *ptrs[:5], 0.1, 0.5, 4, 4, 10, 1) == 1      # islice out of range
    assert f(env, None, 100, 10, 4, *ptrs[:5], 0.1, 0.5, 1, 4, 10, 1) == 1      # window 4 unsupported
    assert f(env, None, 100, 0, 5, *ptrs[:5], 0.1, 0.5, 1, 4, 10, 1) == 0       # nothing to do
    g = lib.Java_edu_berkeley_bid_CUMACH_word2vecNegSlice
    assert g(env, None, 100, 10, 3, 3, *ptrs[:4], 0.1, 0.5, 0, 2, 0, 1) == 1
    assert g(env, None, 100, 10, 5, 5, *ptrs[:4], 0.1, 0.5, 0, 0, 0, 1) == 1    # nslices 0
    e = lib.Java_edu_berkeley_bid_CUMACH_word2vecEvalPosSlice
    assert e(env, None, 100, 10, 5, *ptrs[:6], 0, 2, -1) == 1                   # negative head
    h = lib.Java_edu_berkeley_bid_CUMACH_word2vecEvalNegSlice
    assert h(env, None, 100, 0, 5, 5, *ptrs[:5], 1, 2, 0) == 0
    assert lib.Java_edu_berkeley_bid_CUMACH_w2vCommInitAll(env, None, 0) == 0
    assert lib.Java_edu_berkeley_bid_CUMACH_w2vCommOf(env, None, 0, 0) == 0
    assert lib.Java_edu_berkeley_bid_CUMACH_w2vAllreduceAvg(env, None, 0, ptrs[0], ptrs[1], 10) == 1
    lib.Java_edu_berkeley_bid_CUMACH_w2vCommDestroyAll(env, None, 0)
    assert lib.Java_edu_berkeley_bid_CUMACH_w2vSetSlice(env, None, 0, 0, 2, 0, 1) == 1
