"""Layer files of a QTIP checkpoint (safetensors container): host-side mirror of the quantizer's write_layer_file
(src/pipeline.cpp:314-352 of the reference) and of the runtime's load_linear with its checks
(runtime/src/qtip.cpp:231-289). Arrays are numpy; the work is done by the library (qtip_write_layer_file,
qtip_read_layer_linear)."""
import ctypes as C

import numpy as np

from ._lib import QtipCheckpointLinear, lib


def write_layer_file(path, layer, linears):
    """linears: {name: {"trellis": uint16 [(m/16)(n/16), 32] kernel layout, "SU": bf16 bits uint16 [n],
    "SV": float32 [m] (sign * Wscale), "tlut": fp16 bits uint16 [512, 2], "m": m, "n": n}}."""
    keep = []
    arr = (QtipCheckpointLinear * len(linears))()
    for i, (name, t) in enumerate(linears.items()):
        m, n = int(t["m"]), int(t["n"])
        tr = np.ascontiguousarray(t["trellis"]).view(np.uint16).reshape(-1)
        su = np.ascontiguousarray(t["SU"]).view(np.uint16).reshape(-1)
        sv = np.ascontiguousarray(t["SV"], np.float32).reshape(-1)
        tl = np.ascontiguousarray(t["tlut"]).view(np.uint16).reshape(-1)
        assert tr.size == (m // 16) * (n // 16) * 32 and su.size == n and sv.size == m and tl.size == 1024
        keep += [tr, su, sv, tl]
        arr[i].name, arr[i].m, arr[i].n = name.encode(), m, n
        arr[i].trellis_h, arr[i].su_bf16_h, arr[i].sv_h, arr[i].tlut_h = (a.ctypes.data for a in (tr, su, sv, tl))
    lib().call("qtip_write_layer_file", str(path).encode(), int(layer), arr, len(linears))


def read_layer_linear(path, layer, name, m, n):
    """Returns {"trellis" uint16, "SU" float32, "SV" float32, "tlut" uint16 [512, 2]}; raises QtipError when the file
    violates one of the loader's checks."""
    tr = np.empty(((m // 16) * (n // 16), 32), np.uint16)
    su, sv = np.empty(n, np.float32), np.empty(m, np.float32)
    tl = np.empty((512, 2), np.uint16)
    lib().call("qtip_read_layer_linear", str(path).encode(), int(layer), name.encode(), int(m), int(n),
               tr.ctypes.data_as(C.c_void_p), su.ctypes.data_as(C.c_void_p), sv.ctypes.data_as(C.c_void_p),
               tl.ctypes.data_as(C.c_void_p))
    return {"trellis": tr, "SU": su, "SV": sv, "tlut": tl}
