"""Test infrastructure: runs the UNMODIFIED reference (LightCompress's `llmc` package) end to end --
model adapter, first-block input catcher, `ALGO_REGISTRY[method](...)`, `run_block_loop()`,
`deploy('fake_quant')` -- on a random-init tiny Llama, the way llmc/__main__.py:29-72 drives it.

Nothing of the product imports this file.  It serves three users:
  * tests/golden/make_golden.py, which runs the reference on CPU to write fixtures,
  * the GPU test of the plugin (tests/test_gpu_plugin.py), which runs the reference's own driver
    objects once with its stock classes and once with lightcompress_b200.plugin installed,
  * the CPU test of the plugin, which only constructs.

The reference is looked up in a directory that holds its `llmc` package (`find_reference()`).
`make_ref_copy()` places a verbatim copy of that package plus the four YAML recipes of the hot path
into the git-ignored baseline/_ref/ so that the GPU box, where the checkout itself is absent, can run
the same code.  No reference file is edited: what the reference needs but this image lacks is
supplied from outside, per process:
  * `accelerate` (only `init_empty_weights` is used, base_model.py:10) and `easydict` stubs;
  * `llmc.models` is pre-registered as a bare package pointing at the reference's directory, so that
    `llmc.models.llama` imports without executing llmc/models/__init__.py, which pulls in forty
    adapters and their optional dependencies (librosa, diffusers, ...);
  * on CPU only: `Tensor.cuda` / `Module.cuda` -> identity and `torch.cuda.synchronize` /
    `empty_cache` -> no-ops, which is what the reference's own CI patch (ci_check/change_files.py)
    does by rewriting the sources.
"""
import contextlib
import os
import shutil
import sys
import types

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_COPY = os.path.join(ROOT, 'baseline', '_ref')
HOT_PATH_YAMLS = ('configs/quantization/methods/GPTQ/gptq_w_only.yml',
                  'configs/quantization/methods/Awq/awq_w_only.yml',
                  'configs/quantization/methods/RTN/rtn_w_only.yml',
                  'configs/quantization/backend/vllm/fp8/rtn_fp8.yml')


def make_ref_copy(src, dst=REF_COPY):
    """Verbatim copy of the reference's `llmc` package and the hot path's YAML recipes into `dst`."""
    if not os.path.isdir(os.path.join(src, 'llmc')):
        raise FileNotFoundError(f'{src} holds no llmc package')
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(dst)
    shutil.copytree(os.path.join(src, 'llmc'), os.path.join(dst, 'llmc'),
                    ignore=shutil.ignore_patterns('__pycache__', '*.pyc'))
    for rel in HOT_PATH_YAMLS:
        if os.path.exists(os.path.join(src, rel)):
            os.makedirs(os.path.dirname(os.path.join(dst, rel)), exist_ok=True)
            shutil.copy(os.path.join(src, rel), os.path.join(dst, rel))
    return dst


def find_reference(explicit=None):
    """Directory holding the reference's `llmc` package, or None."""
    for cand in (explicit, os.environ.get('LLMC_REFERENCE_ROOT'), REF_COPY):
        if cand and os.path.isdir(os.path.join(cand, 'llmc')):
            return cand
    return None


class AttrDict(dict):
    """What the reference gets from easydict: attribute access on nested dicts."""

    def __init__(self, d=None, **kw):
        super().__init__()
        for k, v in dict(d or {}, **kw).items():
            self[k] = v

    def __setitem__(self, k, v):
        if isinstance(v, dict) and not isinstance(v, AttrDict):
            v = AttrDict(v)
        super().__setitem__(k, v)

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError:
            raise AttributeError(k) from None

    __setattr__ = __setitem__


_state = {'root': None}


class _CpuTorchProxy:
    """Stands in for the name `torch` inside reference modules that spell out device='cuda' (CPU runs
    only): `torch.device('cuda')` and device= keyword arguments resolve to the CPU."""

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def device(*a, **k):
        return torch.device('cpu')

    @staticmethod
    def tensor(*a, device=None, **k):
        return torch.tensor(*a, **k)

    @staticmethod
    def zeros_like(*a, device=None, **k):
        return torch.zeros_like(*a, **k)


def import_reference(root=None, on_cpu=None):
    """Makes `import llmc...` resolve to the reference under `root`; returns a namespace with the
    modules the drivers below use.  on_cpu (default: no GPU visible) installs the CPU shims."""
    root = find_reference(root)
    if root is None:
        raise FileNotFoundError('no reference checkout: pass its path, set LLMC_REFERENCE_ROOT, or run '
                                'make_ref_copy()')
    if _state['root'] not in (None, root):
        raise RuntimeError(f'the reference was already imported from {_state["root"]}')
    on_cpu = (not torch.cuda.is_available()) if on_cpu is None else on_cpu
    os.environ.setdefault('WORLD_SIZE', '1')
    os.environ.setdefault('RANK', '0')
    os.environ.setdefault('LOCAL_RANK', '0')
    os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
    os.environ.setdefault('MASTER_PORT', '29617')
    import transformers  # noqa: F401  (before the accelerate stub: transformers probes for the real one)
    if 'accelerate' not in sys.modules:
        try:
            import accelerate  # noqa: F401
        except Exception:
            acc = types.ModuleType('accelerate')
            acc.init_empty_weights = contextlib.nullcontext
            sys.modules['accelerate'] = acc
    try:
        import easydict  # noqa: F401
    except ImportError:
        ed = types.ModuleType('easydict')
        ed.EasyDict = AttrDict
        sys.modules['easydict'] = ed
    if on_cpu:
        torch.Tensor.cuda = lambda self, *a, **k: self
        torch.nn.Module.cuda = lambda self, *a, **k: self
        torch.cuda.synchronize = lambda *a, **k: None
        torch.cuda.empty_cache = lambda *a, **k: None
    if root not in sys.path:
        sys.path.insert(0, root)
    if 'llmc.models' not in sys.modules:
        import llmc  # noqa: F401
        pkg = types.ModuleType('llmc.models')
        pkg.__path__ = [os.path.join(root, 'llmc', 'models')]
        pkg.__package__ = 'llmc.models'
        sys.modules['llmc.models'] = pkg
    import torch.distributed as dist
    if not dist.is_initialized():
        # GPTQ.add_batch all-reduces its Hessian (gptq.py:292-295): a one-rank group satisfies it
        dist.init_process_group('gloo' if on_cpu else 'nccl', rank=int(os.environ['RANK']),
                                world_size=int(os.environ['WORLD_SIZE']))
    import llmc.compression.quantization as rquant_pkg
    import llmc.compression.quantization.base_blockwise_quantization as rbase
    import llmc.compression.quantization.gptq as rgptq
    import llmc.compression.quantization.quant as rq
    import llmc.models.llama as rllama
    from llmc.utils.registry_factory import ALGO_REGISTRY
    # The reference recognises norm layers through transformers' ALL_LAYERNORM_LAYERS (module_utils.py:9);
    # the transformers releases it is written for register LlamaRMSNorm there, 5.x no longer does.
    from transformers.models.llama.modeling_llama import LlamaRMSNorm
    from transformers.pytorch_utils import ALL_LAYERNORM_LAYERS
    if LlamaRMSNorm not in ALL_LAYERNORM_LAYERS:
        ALL_LAYERNORM_LAYERS.append(LlamaRMSNorm)
    import llmc.compression.quantization.module_utils as rmu
    if LlamaRMSNorm not in rmu._TRANSFORMERS_LN_TYPES_:
        rmu._TRANSFORMERS_LN_TYPES_.append(LlamaRMSNorm)
    if on_cpu:
        import llmc.compression.quantization.awq as rawq
        import llmc.compression.quantization.spqr as rspqr
        rgptq.torch = _CpuTorchProxy()
        rawq.torch = _CpuTorchProxy()
        rspqr.torch = _CpuTorchProxy()
    _state['root'] = root
    return types.SimpleNamespace(root=root, quant=rq, gptq=rgptq, base=rbase, llama=rllama, pkg=rquant_pkg,
                                 ALGO_REGISTRY=ALGO_REGISTRY, on_cpu=on_cpu)


# ---- a random-init Llama behind the reference's own adapter ------------------------------------------
def tiny_llama_config(hidden=256, inter=512, heads=4, layers=2, vocab=128, max_pos=512):
    from transformers import LlamaConfig
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_attention_heads=heads,
                      num_key_value_heads=heads, num_hidden_layers=layers, vocab_size=vocab,
                      max_position_embeddings=max_pos, rms_norm_eps=1e-5, use_cache=False)
    cfg._attn_implementation = 'sdpa'
    return cfg


def synth_llama_adapter(ref, hf_config, seed=0, dtype=torch.bfloat16):
    """The reference's `Llama` adapter (llmc/models/llama.py) over a random-init LlamaForCausalLM: only
    the two methods that would read a checkpoint from disk are replaced."""
    from transformers import LlamaForCausalLM

    class SynthLlama(ref.llama.Llama):
        def build_tokenizer(self):
            self.tokenizer = None

        def build_model(self):
            self.model_config = hf_config
            model = LlamaForCausalLM(hf_config).to(dtype)
            g = torch.Generator().manual_seed(seed)
            for p in model.parameters():
                p.data = ((torch.randn(p.shape, generator=g) * 0.02) if p.dim() == 2
                          else (1 + 0.1 * torch.randn(p.shape, generator=g))).to(dtype)
            self.model = model

    # on CPU the adapter's own switch keeps the embedding where it is (base_model.py:285-294)
    config = AttrDict(model=dict(type='Llama', path=None, torch_dtype=str(dtype), tokenizer_mode='fast',
                                 use_cpu_to_save_cuda_mem_for_catcher=bool(ref.on_cpu)))
    return SynthLlama(config)


def synth_adapter(ref, family, hf_config, seed=0, dtype=torch.bfloat16):
    """Another of the reference's model adapters over a random-init HF model: family 'opt' (llmc/models/opt.py,
    subsets q/k/v | out_proj | fc1 | fc2) or 'qwen2' (llmc/models/qwen2.py, Llama's layout with biases)."""
    import importlib
    import transformers
    mod = importlib.import_module(f'llmc.models.{family}')
    ref_cls = {'opt': 'Opt', 'qwen2': 'Qwen2', 'llama': 'Llama'}[family]
    hf_cls = {'opt': 'OPTForCausalLM', 'qwen2': 'Qwen2ForCausalLM', 'llama': 'LlamaForCausalLM'}[family]

    class Synth(getattr(mod, ref_cls)):
        def build_tokenizer(self):
            self.tokenizer = None

        def build_model(self):
            self.model_config = hf_config
            model = getattr(transformers, hf_cls)(hf_config).to(dtype).eval()
            g = torch.Generator().manual_seed(seed)
            for n, p in model.named_parameters():
                if p.dim() == 2:
                    p.data = (torch.randn(p.shape, generator=g) * 0.02).to(dtype)
                elif 'norm' in n and n.endswith('weight'):
                    p.data = (1 + 0.1 * torch.randn(p.shape, generator=g)).to(dtype)
                else:
                    p.data = (0.02 * torch.randn(p.shape, generator=g)).to(dtype)
            self.model = model

    Synth.__name__ = ref_cls
    config = AttrDict(model=dict(type=ref_cls, path=None, torch_dtype=str(dtype), tokenizer_mode='fast',
                                 use_cpu_to_save_cuda_mem_for_catcher=bool(ref.on_cpu)))
    return Synth(config)


def gptq_quant_config(special=None, bit=4, symmetric=False, quant_out=True):
    """`quant` section of configs/quantization/methods/GPTQ/gptq_w_only.yml (values restated: W4 g128,
    actorder, static_groups False, percdamp 0.01, blocksize 128, true_sequential, quant_out)."""
    sp = dict(actorder=True, static_groups=False, percdamp=0.01, blocksize=128, true_sequential=True)
    sp.update(special or {})
    return AttrDict(method='GPTQ', modality='language', quant_out=quant_out,
                    weight=dict(bit=bit, symmetric=symmetric, granularity='per_group', group_size=128),
                    special=sp)


def gptq_w8a8_quant_config():
    """`quant` section of configs/quantization/backend/vllm/w8a8_combin/step_2_gptq.yml (values restated:
    W8 symmetric per_channel, A8 symmetric per_token, static_groups, actorder)."""
    return AttrDict(method='GPTQ', modality='language', quant_out=True,
                    weight=dict(bit=8, symmetric=True, granularity='per_channel', group_size=-1, qmax_to_tensor=True,
                                calib_algo='minmax'),
                    act=dict(bit=8, symmetric=True, granularity='per_token', qmax_to_tensor=True, calib_algo='minmax'),
                    special=dict(actorder=True, static_groups=True, percdamp=0.01, blocksize=128, true_sequential=True,
                                 online_rotate=False, fp32_had=True))


def spqr_quant_config(special=None, quant_out=True):
    """`quant` section of configs/quantization/methods/SpQR/spqr_w_only.yml (values restated: W4 groups of
    16, round_zp False, actorder, percdamp 1, blocksize 128, relative_threshold 0.2, 3-bit second-level
    statistics in groups of 16)."""
    stat = dict(bit=3, symmetric=False, granularity='per_group', group_size=16, round_zp=False)
    sp = dict(actorder=True, percdamp=1, blocksize=128, true_sequential=True, relative_threshold=0.2,
              simplified_outliers=False, scale=dict(stat), zero=dict(stat))
    sp.update(special or {})
    return AttrDict(method='SpQR', modality='language', quant_out=quant_out,
                    weight=dict(bit=4, symmetric=False, granularity='per_group', group_size=16, round_zp=False),
                    special=sp)


def awq_quant_config(symmetric=True, quant_out=True):
    """`quant` section of configs/quantization/methods/Awq/awq_w_only.yml (values restated: W4 g128
    symmetric, trans v2, weight_clip, clip_sym)."""
    return AttrDict(method='Awq', modality='language', quant_out=quant_out,
                    weight=dict(bit=4, symmetric=symmetric, granularity='per_group', group_size=128),
                    special=dict(trans=True, trans_version='v2', weight_clip=True, clip_sym=symmetric))


def rtn_quant_config(bit=4, symmetric=False):
    return AttrDict(method='RTN', modality='language',
                    weight=dict(bit=bit, symmetric=symmetric, granularity='per_group', group_size=128))


def calib_ids(n_samples, seq_len, vocab, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [{'input_ids': torch.randint(0, vocab, (1, seq_len), generator=g)} for _ in range(n_samples)]


def run_algorithm(ref, model, quant_cfg, calib, seq_len, deploy='fake_quant'):
    """llmc/__main__.py:55-74 for one modality: catch the first block's inputs, construct the registered
    algorithm, run its block loop, deploy.  Returns the algorithm object."""
    config = AttrDict(model=dict(type='Llama'), calib=dict(bs=1, seq_len=seq_len, n_samples=len(calib) if calib else 0),
                      quant=quant_cfg, base=dict(seed=0))
    if quant_cfg.method == 'RTN':
        algo = ref.ALGO_REGISTRY['RTN'](model, quant_cfg, None, None, config)
    else:
        model.collect_first_block_input(calib, None)
        algo = ref.ALGO_REGISTRY[quant_cfg.method](model, quant_cfg, model.get_first_block_input(), None, config)
    algo.run_block_loop()
    if deploy:
        algo.deploy(deploy)
    return algo


def linear_state(model):
    """Per block and linear: the tensors GPTQ leaves (weight + buf_*), moved to the CPU."""
    out = []
    for block in model.get_blocks():
        d = {}
        for name, m in block.named_modules():
            if hasattr(m, 'weight') and m.weight is not None and m.weight.dim() == 2:
                e = {'weight': m.weight.data.detach().cpu().clone()}
                for k, b in m.named_buffers(recurse=False):
                    if k.startswith('buf_'):
                        e[k] = b.detach().cpu().clone()
                d[name] = e
        out.append(d)
    return out
