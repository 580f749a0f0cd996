"""Host-side mirror of the reference RTN algorithm's hot methods.

RTN has no calibration transform (llmc/compression/quantization/rtn.py:10-28); all its work is
the dynamic weight / activation fake quant that `deploy` wires into the replacement linears
(base_blockwise_quantization.py:50-86: w_qdq, w_q, a_qdq).
"""
import torch


class RTN:
    def __init__(self, wquantizer, aquantizer=None):
        self.wquantizer = wquantizer
        self.aquantizer = aquantizer

    @torch.no_grad()
    def w_qdq(self, module, wquantizer=None):
        return (wquantizer or self.wquantizer).fake_quant_weight_dynamic(module.weight.data)

    @torch.no_grad()
    def w_q(self, module, wquantizer=None):
        return (wquantizer or self.wquantizer).real_quant_weight_dynamic(module.weight.data)

    @torch.no_grad()
    def a_qdq(self, act, module=None, aquantizer=None, input_index=0):
        return (aquantizer or self.aquantizer).fake_quant_act_dynamic(act)
