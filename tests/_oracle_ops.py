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
