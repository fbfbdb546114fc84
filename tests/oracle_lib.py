"""ctypes access to the checkers: oracle/liboracle.so (the C restatement) and, when it has
been built, oracle/_ref/libtf_ref.so (the unmodified reference behind a C shim).

Test infrastructure only: nothing in the product imports this module.
"""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "liboracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libtf_ref.so")

_f = ctypes.POINTER(ctypes.c_float)
_d = ctypes.POINTER(ctypes.c_double)
_l = ctypes.POINTER(ctypes.c_int64)
_i64 = ctypes.c_int64
_int = ctypes.c_int


def _build_oracle():
    src = os.path.join(ORACLE_DIR, "oracle.c")
    if os.path.exists(ORACLE_SO) and os.path.getmtime(ORACLE_SO) >= os.path.getmtime(src):
        return
    subprocess.run(["make", "-C", ORACLE_DIR, os.path.join(ORACLE_DIR, "liboracle.so")], check=True,
                   capture_output=True)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def fp(a):
    return a.ctypes.data_as(_f) if a is not None else None


def lp(a):
    return a.ctypes.data_as(_l) if a is not None else None


class Oracle:
    def __init__(self):
        _build_oracle()
        self.lib = ctypes.CDLL(ORACLE_SO)
        L = self.lib
        L.orc_nll_mean.restype = ctypes.c_float
        L.orc_mlp_grads.restype = ctypes.c_float
        L.orc_im2col_index.restype = _i64
        L.orc_conv_out_dim.restype = _i64
        L.orc_round_bf16.restype = ctypes.c_float
        L.orc_get_threads.restype = _int

    # -- contraction ----------------------------------------------------------------------
    def matmul(self, A, B, mt=True):
        A, B = f32(A), f32(B)
        M, K = A.shape
        K2, N = B.shape
        assert K == K2
        C = np.empty((M, N), np.float32)
        fn = self.lib.orc_matmul_f32_mt if mt else self.lib.orc_matmul_f32
        fn(fp(A), fp(B), fp(C), _i64(M), _i64(N), _i64(K))
        return C

    def matmul_f64(self, A, B):
        A, B = f32(A), f32(B)
        M, K = A.shape
        N = B.shape[1]
        C = np.empty((M, N), np.float64)
        self.lib.orc_matmul_f64(fp(A), fp(B), C.ctypes.data_as(_d), _i64(M), _i64(N), _i64(K))
        return C

    def matmul_rows(self, A, B, rows):
        A, B = f32(A), f32(B)
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        K, N = B.shape
        out = np.empty((len(rows), N), np.float32)
        self.lib.orc_matmul_f32_rows(fp(A), fp(B), fp(out), lp(rows), _i64(len(rows)), _i64(N), _i64(K))
        return out

    def matmul_cols(self, A, B, cols):
        A, B = f32(A), f32(B)
        cols = np.ascontiguousarray(cols, dtype=np.int64)
        M, K = A.shape
        N = B.shape[1]
        out = np.empty((M, len(cols)), np.float32)
        self.lib.orc_matmul_f32_cols(fp(A), fp(B), fp(out), lp(cols), _i64(len(cols)), _i64(M), _i64(N),
                                     _i64(K))
        return out

    def round_bf16(self, a):
        a = f32(a)
        out = np.empty_like(a)
        self.lib.orc_round_bf16_array(fp(a), fp(out), _i64(a.size))
        return out

    def matmul_backward(self, A, B, G):
        """dA = G·Bᵀ, dB = Aᵀ·G in the reference's order (transposes then Tensor::matmul)."""
        A, B, G = f32(A), f32(B), f32(G)
        return self.matmul(G, np.ascontiguousarray(B.T)), self.matmul(np.ascontiguousarray(A.T), G)

    # -- linear ------------------------------------------------------------------------------
    def linear_forward(self, X, W, bias=None, relu=False):
        X, W = f32(X), f32(W)
        b = f32(bias) if bias is not None else None
        batch, in_f = X.shape
        out_f = W.shape[0]
        Y = np.empty((batch, out_f), np.float32)
        self.lib.orc_linear_forward(fp(X), fp(W), fp(b), fp(Y), _i64(batch), _i64(in_f), _i64(out_f),
                                    _int(int(relu)))
        return Y

    def linear_backward(self, X, W, Y, dY, relu=False):
        X, W, Y, dY = f32(X), f32(W), f32(Y), f32(dY)
        batch, in_f = X.shape
        out_f = W.shape[0]
        dX = np.empty((batch, in_f), np.float32)
        dW = np.empty((out_f, in_f), np.float32)
        db = np.empty((out_f,), np.float32)
        self.lib.orc_linear_backward(fp(X), fp(W), fp(Y), fp(dY), fp(dX), fp(dW), fp(db), _i64(batch),
                                     _i64(in_f), _i64(out_f), _int(int(relu)))
        return dX, dW, db

    # -- convolution ---------------------------------------------------------------------------
    def conv_out_dim(self, n, k, s, p, d):
        return int(self.lib.orc_conv_out_dim(_i64(n), _i64(k), _i64(s), _i64(p), _i64(d)))

    def im2col_index_range(self, first, count, C, H, W, kH, kW, sh, sw, ph, pw, dh, dw):
        outH, outW = self.conv_out_dim(H, kH, sh, ph, dh), self.conv_out_dim(W, kW, sw, pw, dw)
        out = np.empty((count,), np.int64)
        self.lib.orc_im2col_index_range(_i64(first), _i64(count), lp(out), *[_i64(v) for v in (
            C, H, W, kH, kW, sh, sw, ph, pw, dh, dw, outH, outW)])
        return out

    def im2col(self, x, kH, kW, sh, sw, ph, pw, dh, dw):
        x = f32(x)
        N, C, H, W = x.shape
        outH, outW = self.conv_out_dim(H, kH, sh, ph, dh), self.conv_out_dim(W, kW, sw, pw, dw)
        col = np.empty((N, C * kH * kW, outH * outW), np.float32)
        self.lib.orc_im2col_f32(fp(x), fp(col), *[_i64(v) for v in (N, C, H, W, kH, kW, sh, sw, ph, pw, dh, dw)])
        return col

    def conv2d_forward(self, x, w, bias, stride=(1, 1), pad=(0, 0), dil=(1, 1), via_im2col=False):
        x, w = f32(x), f32(w)
        b = f32(bias) if bias is not None else None
        N, C, H, W = x.shape
        Cout, _, kH, kW = w.shape
        outH, outW = self.conv_out_dim(H, kH, stride[0], pad[0], dil[0]), self.conv_out_dim(W, kW, stride[1], pad[1], dil[1])
        out = np.empty((N, Cout, outH, outW), np.float32)
        fn = self.lib.orc_conv2d_forward_im2col if via_im2col else self.lib.orc_conv2d_forward
        fn(fp(x), fp(w), fp(b), fp(out), *[_i64(v) for v in (
            N, C, H, W, Cout, kH, kW, stride[0], stride[1], pad[0], pad[1], dil[0], dil[1])])
        return out

    def conv2d_backward(self, x, w, dY, stride=(1, 1), pad=(0, 0), dil=(1, 1)):
        x, w, dY = f32(x), f32(w), f32(dY)
        N, C, H, W = x.shape
        Cout, _, kH, kW = w.shape
        gi = np.empty_like(x)
        gw = np.empty_like(w)
        gb = np.empty((Cout,), np.float32)
        self.lib.orc_conv2d_backward(fp(x), fp(w), fp(dY), fp(gi), fp(gw), fp(gb), *[_i64(v) for v in (
            N, C, H, W, Cout, kH, kW, stride[0], stride[1], pad[0], pad[1], dil[0], dil[1])])
        return gi, gw, gb

    # -- loss / optimiser / MLP -------------------------------------------------------------------
    def log_softmax(self, x):
        x = f32(x)
        y = np.empty_like(x)
        self.lib.orc_log_softmax(fp(x), fp(y), _i64(x.shape[0]), _i64(x.shape[1]))
        return y

    def nll_mean(self, logits, labels, global_rows=None):
        logits = f32(logits)
        labels = np.ascontiguousarray(labels, dtype=np.int64)
        dz = np.empty_like(logits)
        rows, cols = logits.shape
        loss = self.lib.orc_nll_mean(fp(logits), lp(labels), fp(dz), _i64(rows), _i64(cols),
                                     _i64(global_rows or rows))
        return float(loss), dz

    def sgd_momentum(self, p, v, g, lr, mu):
        p, v, g = f32(p).copy(), f32(v).copy(), f32(g)
        self.lib.orc_sgd_momentum(fp(p), fp(v), fp(g), _i64(p.size), ctypes.c_float(lr), ctypes.c_float(mu))
        return p, v

    def mlp_grads(self, X, labels, Ws, bs=None, global_rows=None):
        X = f32(X)
        labels = np.ascontiguousarray(labels, dtype=np.int64)
        Ws = [f32(w) for w in Ws]
        bs = [f32(b) for b in bs] if bs is not None else [None, None, None]
        batch, d0 = X.shape
        d1, d2, d3 = Ws[0].shape[0], Ws[1].shape[0], Ws[2].shape[0]
        dWs = [np.empty_like(w) for w in Ws]
        dbs = [np.empty((w.shape[0],), np.float32) for w in Ws]
        loss = self.lib.orc_mlp_grads(fp(X), lp(labels), _i64(batch), _i64(global_rows or batch), _i64(d0),
                                      _i64(d1), _i64(d2), _i64(d3), fp(Ws[0]), fp(bs[0]), fp(Ws[1]),
                                      fp(bs[1]), fp(Ws[2]), fp(bs[2]), fp(dWs[0]), fp(dbs[0]), fp(dWs[1]),
                                      fp(dbs[1]), fp(dWs[2]), fp(dbs[2]))
        return float(loss), dWs, dbs


class Reference:
    """The unmodified reference CPU implementation behind oracle/ref_shim.cpp."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.lib = ctypes.CDLL(REF_SO)
        self.lib.ref_last_error.restype = ctypes.c_char_p

    def _ok(self, rc):
        if rc != 0:
            raise RuntimeError("reference threw: " + self.lib.ref_last_error().decode())

    def matmul(self, A, B):
        A, B = f32(A), f32(B)
        M, K = A.shape
        N = B.shape[1]
        C = np.empty((M, N), np.float32)
        self._ok(self.lib.ref_matmul(fp(A), fp(B), fp(C), _i64(M), _i64(N), _i64(K)))
        return C

    def hold_matrix(self, B):
        B = f32(B)
        self.lib.ref_hold_matrix.restype = ctypes.c_void_p
        h = self.lib.ref_hold_matrix(fp(B), _i64(B.shape[0]), _i64(B.shape[1]))
        if not h:
            raise RuntimeError("reference threw: " + self.lib.ref_last_error().decode())
        return (ctypes.c_void_p(h), B.shape)

    def matmul_held(self, A, held):
        A = f32(A)
        handle, (K, N) = held
        C = np.empty((A.shape[0], N), np.float32)
        self._ok(self.lib.ref_matmul_held(fp(A), handle, fp(C), _i64(A.shape[0])))
        return C

    def matmul_backward(self, A, B, G):
        A, B, G = f32(A), f32(B), f32(G)
        M, K = A.shape
        N = B.shape[1]
        dA, dB = np.empty_like(A), np.empty_like(B)
        self._ok(self.lib.ref_matmul_backward(fp(A), fp(B), fp(G), fp(dA), fp(dB), _i64(M), _i64(N), _i64(K)))
        return dA, dB

    def linear_weight(self, in_f, out_f):
        W = np.empty((out_f, in_f), np.float32)
        self._ok(self.lib.ref_linear_weight(_int(in_f), _int(out_f), fp(W)))
        return W

    def linear_fwd_bwd(self, X, W, G, relu):
        X = f32(X)
        batch, in_f = X.shape
        W = f32(W)
        out_f = W.shape[0]
        Y = np.empty((batch, out_f), np.float32)
        dX = np.empty_like(X)
        dW = np.empty_like(W)
        G = f32(G)
        self._ok(self.lib.ref_linear_fwd_bwd(fp(X), fp(W), fp(G), _i64(batch), _int(in_f), _int(out_f),
                                             _int(int(relu)), fp(Y), fp(dX), fp(dW)))
        return Y, dX, dW

    def conv_weight(self, cin, cout, k):
        W = np.empty((cout, cin, k, k), np.float32)
        self._ok(self.lib.ref_conv_weight(_int(cin), _int(cout), _int(k), fp(W)))
        return W

    def conv2d_forward(self, X, W, stride, pad, dil):
        X, W = f32(X), f32(W)
        N, C, H, Wd = X.shape
        cout, _, k, _ = W.shape
        oh = (H + 2 * pad - dil * (k - 1) - 1) // stride + 1
        ow = (Wd + 2 * pad - dil * (k - 1) - 1) // stride + 1
        out = np.empty((N, cout, oh, ow), np.float32)
        self._ok(self.lib.ref_conv2d_forward(fp(X), fp(W), _i64(N), _int(C), _i64(H), _i64(Wd), _int(cout),
                                             _int(k), _int(stride), _int(pad), _int(dil), fp(out)))
        return out

    def log_softmax(self, X):
        X = f32(X)
        out = np.empty_like(X)
        self._ok(self.lib.ref_log_softmax(fp(X), _i64(X.shape[0]), _i64(X.shape[1]), fp(out)))
        return out

    def mlp_grads(self, X, labels, Ws):
        X = f32(X)
        labels = np.ascontiguousarray(labels, dtype=np.int64)
        Ws = [f32(w) for w in Ws]
        batch, d0 = X.shape
        d1, d2, d3 = Ws[0].shape[0], Ws[1].shape[0], Ws[2].shape[0]
        loss = ctypes.c_float(0)
        dWs = [np.empty_like(w) for w in Ws]
        self._ok(self.lib.ref_mlp_grads(fp(X), lp(labels), _i64(batch), _int(d0), _int(d1), _int(d2), _int(d3),
                                        fp(Ws[0]), fp(Ws[1]), fp(Ws[2]), ctypes.byref(loss), fp(dWs[0]),
                                        fp(dWs[1]), fp(dWs[2])))
        return float(loss.value), dWs


def have_reference():
    return os.path.exists(REF_SO)
