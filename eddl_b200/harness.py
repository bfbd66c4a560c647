"""Python binding of the net harness (``eddl_b200/host/net_harness.cpp``).

``NetHarness(libpath, ...)`` drives an EDDL net built through EDDL's own public API.  With
the drop-in library (``baseline/_ref/libeddl_b200_dropin.so``: EDDL's host code compiled with
``-DcGPU`` on top of this backend) the net runs on ``CS_GPU``; the tests also hand it the CPU
build of the reference to obtain the values to compare against.
"""
import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROPIN = os.path.join(ROOT, "baseline", "_ref", "libeddl_b200_dropin.so")

_f32p = ctypes.c_void_p


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


class HarnessError(RuntimeError):
    pass


def load(path=DROPIN):
    if not os.path.exists(path):
        raise ImportError("eddl_b200: %s is missing -- build it with `python eddl_b200/build.py dropin` "
                          "(needs the EDDL source tree)" % path)
    cdll = ctypes.CDLL(path)
    cdll.ebh_last_error.restype = ctypes.c_char_p
    return cdll


class NetHarness:
    def __init__(self, cdll, config, device=0, hw=0, classes=0, threads=-1, optimizer="sgd", lr=0.01, mu=0.9,
                 loss="categorical_cross_entropy"):
        self.L, self.h = cdll, ctypes.c_int(0)
        self._ck(self.L.ebh_create(config.encode(), hw, classes, device, threads, optimizer.encode(),
                                   ctypes.c_float(lr), ctypes.c_float(mu), loss.encode(), ctypes.byref(self.h)))
        nt, nf = ctypes.c_int(), ctypes.c_longlong()
        self._ck(self.L.ebh_num_params(self.h, ctypes.byref(nt), ctypes.byref(nf)))
        self.ntensors, self.nfloats = nt.value, nf.value
        self.device = device

    def _ck(self, st):
        if st != 0:
            raise HarnessError(self.L.ebh_last_error().decode())

    def param_info(self):
        out = []
        for i in range(self.ntensors):
            nd, shape, name = ctypes.c_int(), (ctypes.c_int * 4)(), ctypes.create_string_buffer(64)
            self._ck(self.L.ebh_param_info(self.h, i, ctypes.byref(nd), shape, name))
            out.append((name.value.decode(), tuple(shape[:nd.value])))
        return out

    def set_params(self, flat):
        flat = np.ascontiguousarray(flat, dtype=np.float32)
        assert flat.size == self.nfloats
        self._ck(self.L.ebh_set_params(self.h, _ptr(flat)))

    def get_params(self):
        flat = np.empty(self.nfloats, dtype=np.float32)
        self._ck(self.L.ebh_get_params(self.h, _ptr(flat)))
        return flat

    def train_batch(self, x, y, nocopy=False):
        x = np.ascontiguousarray(x, dtype=np.float32); y = np.ascontiguousarray(y, dtype=np.float32)
        loss, acc = ctypes.c_float(), ctypes.c_float()
        f = self.L.ebh_train_batch_nocopy if nocopy else self.L.ebh_train_batch
        self._ck(f(self.h, _ptr(x), _ptr(y), x.shape[0], ctypes.byref(loss), ctypes.byref(acc)))
        return loss.value, acc.value

    def train_fine(self, x, y):
        """One step as zeroGrads / forward / backward / update instead of train_batch."""
        x = np.ascontiguousarray(x, dtype=np.float32); y = np.ascontiguousarray(y, dtype=np.float32)
        loss, acc = ctypes.c_float(), ctypes.c_float()
        self._ck(self.L.ebh_train_fine(self.h, _ptr(x), _ptr(y), x.shape[0], ctypes.byref(loss), ctypes.byref(acc)))
        return loss.value, acc.value

    def save(self, path):
        self._ck(self.L.ebh_save(self.h, os.fsencode(path)))

    def load(self, path):
        self._ck(self.L.ebh_load(self.h, os.fsencode(path)))

    def train_resident(self, steps):
        loss = ctypes.c_float()
        self._ck(self.L.ebh_train_resident(self.h, steps, ctypes.byref(loss)))
        return loss.value

    def local_step(self):
        """One step on the resident batch without cross-rank averaging."""
        self._ck(self.L.ebh_local_step(self.h))

    def forward(self, x, classes):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty((x.shape[0], classes), dtype=np.float32)
        self._ck(self.L.ebh_forward(self.h, _ptr(x), x.shape[0], _ptr(out)))
        return out

    def num_layers(self):
        n = ctypes.c_int()
        self._ck(self.L.ebh_num_layers(self.h, ctypes.byref(n)))
        return n.value

    def layer_name(self, i):
        name = ctypes.create_string_buffer(64)
        self._ck(self.L.ebh_layer_name(self.h, i, name))
        return name.value.decode()

    def layer_tensor(self, i, what=0):
        size = ctypes.c_longlong()
        self._ck(self.L.ebh_layer_tensor(self.h, i, what, None, ctypes.c_longlong(0), ctypes.byref(size)))
        out = np.empty(size.value, dtype=np.float32)
        self._ck(self.L.ebh_layer_tensor(self.h, i, what, _ptr(out), ctypes.c_longlong(out.size), ctypes.byref(size)))
        return out

    # distributed (GPU build only)
    def broadcast_params(self):
        self._ck(self.L.ebh_broadcast_params(self.h))

    def avg_weights(self, curr_batch=1, batches_per_avg=1):
        self._ck(self.L.ebh_avg_weights(self.h, curr_batch, batches_per_avg))

    def sync(self):
        self._ck(self.L.ebh_sync(self.h))

    def close(self):
        if self.h.value:
            self.L.ebh_destroy(self.h)
            self.h = ctypes.c_int(0)


def init_weights(info, seed, mode="glorot_uniform"):
    """Seeded initial parameters for a net, in the harness's flat order.

    EDDL's initialisers ignore their seed, so parity runs inject weights.  Distributions follow
    EDDL's definitions: Glorot uniform limit sqrt(6/(fan_in+fan_out)) with conv fans kr*kc*C and
    kr*kc*K (src/initializers/initializer_glorot_uniform.cpp:50-60); He normal std sqrt(2/fan_in)
    (initializer_he_normal.cpp:38-42).  Biases 0; BatchNorm gamma 1, beta 0, running mean 0,
    running variance 0 (LBatchNorm::initialize, src/layers/normalization/layer_batchnorm.cpp:50-57,154-159).
    A layer's 1-D tensors are recognised by name: batchnorm layers own (gamma, beta, mean, variance).
    """
    rng = np.random.default_rng(seed)
    chunks, bn_seen = [], {}
    for name, shape in info:
        n = int(np.prod(shape))
        if len(shape) == 4:
            k, c, kr, kc = shape
            fan_in, fan_out = kr * kc * c, kr * kc * k
        elif len(shape) == 2:
            fan_in, fan_out = shape
        else:
            if "batchnorm" in name.lower() or name.lower().startswith("bn"):
                idx = bn_seen.get(name, 0); bn_seen[name] = idx + 1
                chunks.append(np.ones(n, np.float32) if idx == 0 else np.zeros(n, np.float32))
            else:
                chunks.append(np.zeros(n, np.float32))
            continue
        if mode == "glorot_uniform":
            lim = np.sqrt(6.0 / (fan_in + fan_out))
            chunks.append(rng.uniform(-lim, lim, n).astype(np.float32))
        else:
            chunks.append((rng.standard_normal(n) * np.sqrt(2.0 / fan_in)).astype(np.float32))
    return np.concatenate(chunks)
