"""Model / run configurations and the reference's published regression numbers for the language-model benchmarks.

The numbers in ``get_golden_*_stats`` were measured by the reference project on its CI machines (4 x 16 GB GPUs of an
older generation; benchmarks/golden_configs/lm_wikitext2.py:11-163); they are kept as the bar to clear.
"""

import torch.nn as nn


def _lm(ninp=2048, nhid=2048, layers=10, seq_len=32, **extra):
    cfg = {"vocab_size": 10000, "ninp": ninp, "nhid": nhid, "nhead": 32, "dropout": 0, "initrange": 0.1, "clip_value": 0.05,
           "num_decoder_layers": layers, "seq_len": seq_len}
    cfg.update(extra)
    return cfg


def _run(batch_size=8, **extra):
    cfg = {"epochs": 1, "lr": 0.001, "batch_size": batch_size, "criterion": nn.CrossEntropyLoss()}
    cfg.update(extra)
    return cfg


class Offload_Transformer:
    get_model_config = staticmethod(lambda: _lm())
    get_benchmark_config = staticmethod(lambda checkpoint_activation=True: _run(
        checkpoint_activation=checkpoint_activation, num_microbatches=1, slices=3))
    get_golden_real_stats = staticmethod(lambda: {"avg_wps": 192.105, "std_dev_wps": 39.56, "peak_mem_usage": 1180848128})


class Offload_Sequential:
    get_model_config = staticmethod(lambda: {"inputs": 100, "outputs": 5, "hidden": 1000, "layers": 100, "clip_value": 0.05})
    get_benchmark_config = staticmethod(lambda: _run(slices=3, checkpoint_activation=True, num_microbatches=1))


class FSDP:
    get_model_config = staticmethod(lambda: _lm())
    get_benchmark_config = staticmethod(lambda: _run())
    get_golden_synthetic_stats = staticmethod(lambda: {"avg_wps": 486.303, "std_dev_wps": 71.307, "peak_mem_usage": [5.5055 * 2**30] * 4})

    @staticmethod
    def get_golden_real_stats():
        raise NotImplementedError("Real-data benchmarks need the wikitext-2 corpus, which is not bundled.")


class Pipe:
    get_model_config = staticmethod(lambda: _lm())
    get_benchmark_config = staticmethod(lambda: _run())
    get_golden_real_stats = staticmethod(lambda: {"avg_wps": 703.778, "std_dev_wps": 5.732,
                                                  "peak_mem_usage": [2320996352, 1396742144, 1396742144, 2340010496]})


class MOE:
    # (seq_len - 1) must be divisible by num_local_experts
    get_model_config = staticmethod(lambda: _lm(ninp=1024, nhid=4096, layers=20, seq_len=33, is_moe=True, num_local_experts=2))
    get_benchmark_config = staticmethod(lambda: _run(batch_size=32))
