"""Stand-in "local kernels" for the sequence-parallel host logic, backed by the CPU oracle.

Test infrastructure: lets the exchange/carry logic of ``scanscam_b200.sharded`` run on CPU
process groups.  The interface is the one ``sharded.CudaShardOps`` implements.
"""
import numpy as np
import torch

import oracle


class OracleShardOps:
    @staticmethod
    def reduce_forward(gate, value):
        a, b = gate.numpy(), value.numpy()
        h = oracle.scan_forward(a, b)
        # A = running product in sequence order, B = last value of the scan started from zero
        A = np.ones(a.shape[0], a.dtype)
        for t in range(a.shape[1]):
            A = A * a[:, t]
        return torch.from_numpy(np.stack([A, h[:, -1]], axis=1).astype(a.dtype))

    @staticmethod
    def reduce_backward(gate, out_grad):
        a, g = gate.numpy(), out_grad.numpy()
        A = np.ones(a.shape[0], a.dtype)
        D = np.zeros(a.shape[0], a.dtype)
        for t in range(a.shape[1] - 1, -1, -1):
            D = a[:, t] * (g[:, t] + D)
            A = A * a[:, t]
        return torch.from_numpy(np.stack([A, D], axis=1).astype(a.dtype))

    @staticmethod
    def map_forward(gate, value, cut=0.0, walked=None):
        """(A, B) folded from the shard's last step backwards; a row stops once |A| <= cut."""
        a, b = gate.numpy(), value.numpy()
        A = np.ones(a.shape[0], a.dtype)
        B = np.zeros(a.shape[0], a.dtype)
        live = np.ones(a.shape[0], bool)
        steps = 0
        for t in range(a.shape[1] - 1, -1, -1):
            if not live.any():
                break
            # prepend element t: h_end = A*(a_t*h + b_t) + B
            B = np.where(live, A * b[:, t] + B, B)
            A = np.where(live, A * a[:, t], A)
            steps += int(live.sum())
            live &= ~(np.abs(A) <= cut)
        if walked is not None:
            walked += steps
        return torch.from_numpy(np.stack([A, B], axis=1).astype(a.dtype))

    @staticmethod
    def map_backward(gate, out_grad, cut=0.0, walked=None):
        """(A, D) of c_t = a_t*(g_t + c_{t+1}) folded from the shard's first step forwards."""
        a, g = gate.numpy(), out_grad.numpy()
        A = np.ones(a.shape[0], a.dtype)
        D = np.zeros(a.shape[0], a.dtype)
        live = np.ones(a.shape[0], bool)
        steps = 0
        for t in range(a.shape[1]):
            if not live.any():
                break
            # append element t: c_first = A*(a_t*(g_t + c)) + D
            D = np.where(live, (A * a[:, t]) * g[:, t] + D, D)
            A = np.where(live, A * a[:, t], A)
            steps += int(live.sum())
            live &= ~(np.abs(A) <= cut)
        if walked is not None:
            walked += steps
        return torch.from_numpy(np.stack([A, D], axis=1).astype(a.dtype))

    @staticmethod
    def carry(aggs, shard, reverse):
        m = aggs.numpy()
        x = np.zeros(m.shape[1], m.dtype)
        order = range(shard) if not reverse else range(m.shape[0] - 1, shard, -1)
        for s in order:
            x = m[s, :, 0] * x + m[s, :, 1]
        return torch.from_numpy(x.astype(m.dtype))

    @staticmethod
    def scan_forward(gate, value, h_in):
        return torch.from_numpy(oracle.scan_forward(gate.numpy(), value.numpy(), h_in=h_in.numpy()))

    @staticmethod
    def scan_backward(gate, output, out_grad, c_in, h_prev):
        ga, gb = oracle.scan_backward(gate.numpy(), output.numpy(), out_grad.numpy(),
                                      gb_in=c_in.numpy(), h_prev=h_prev.numpy())
        return torch.from_numpy(ga), torch.from_numpy(gb)
