"""DeepSpeed-style front end.

``from msamp import deepspeed`` is meant as a drop-in for ``import deepspeed``: when DeepSpeed is
installed its public names are re-exported here (as the reference does, msamp/deepspeed/__init__.py:10),
and ``initialize`` builds MS-AMP engines from the same JSON configuration with an extra section::

    "msamp": {"enabled": true, "opt_level": "O1|O2|O3", "use_te": false}

With DeepSpeed installed, ``initialize`` returns a subclass of its ``DeepSpeedEngine`` whose optimizer is one of msamp's FP8
wrappers (``runtime/adapter.py``).  Without it, the stand-alone engines below are used; they do not depend on DeepSpeed: ``MSAMPDeepSpeedEngine`` implements the training-loop
surface (``engine(inputs)``, ``engine.backward(loss)``, ``engine.step()``, checkpoints, gradient
accumulation, clipping, loss scaling, ZeRO stages 0-2 and pipeline parallelism) on msamp's own optimizers
and fused collectives.
"""
try:    # pragma: no cover - DeepSpeed is optional
    from deepspeed import *    # noqa: F401,F403
except Exception:
    pass

import json

import torch

from msamp.deepspeed.runtime.config import MSAMPDeepSpeedConfig
from msamp.deepspeed.runtime.engine import MSAMPDeepSpeedEngine
from msamp.deepspeed.runtime.pipe.engine import MSAMPPipelineEngine, PipelineModule


def initialize(args=None, model=None, optimizer=None, model_parameters=None, training_data=None, lr_scheduler=None, mpu=None,
               dist_init_required=None, collate_fn=None, config=None, config_params=None):
    """Build an engine. Returns ``(engine, optimizer, training_dataloader, lr_scheduler)``.

    ``config`` is a dict or the path of a JSON file (``args.deepspeed_config`` is used when it is missing).
    """
    if model is None:
        raise AssertionError('deepspeed.initialize requires a model')
    if config is None:
        config = config_params
    if config is None and args is not None:
        config = getattr(args, 'deepspeed_config', None)
    if config is None:
        raise AssertionError('DeepSpeed requires --deepspeed_config to specify configuration file')
    if isinstance(config, str):
        with open(config) as f:
            config = json.load(f)
    if dist_init_required and not torch.distributed.is_initialized():
        import os
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29500')
        torch.distributed.init_process_group('nccl' if torch.cuda.is_available() else 'gloo')
    from msamp.deepspeed.runtime import adapter
    if adapter.deepspeed_available() and not isinstance(model, PipelineModule):
        # DeepSpeed is installed: its own engine and config, subclassed so that the optimizer is msamp's
        engine_cls, config_cls = adapter.make_engine_class(), adapter.make_config_class()
        cfg = config_cls(config, mpu)
        engine = engine_cls(args=args, model=model, optimizer=optimizer, model_parameters=model_parameters, training_data=training_data,
                            lr_scheduler=lr_scheduler, mpu=mpu, dist_init_required=dist_init_required, collate_fn=collate_fn, config=config,
                            config_class=cfg)
        return engine, engine.optimizer, engine.training_dataloader, engine.lr_scheduler
    if mpu is None and isinstance(model, PipelineModule):
        mpu = model    # batch arithmetic counts data-parallel replicas, not pipeline stages
    cfg = MSAMPDeepSpeedConfig(config, mpu)
    cls = MSAMPPipelineEngine if isinstance(model, PipelineModule) else MSAMPDeepSpeedEngine
    engine = cls(args=args, model=model, optimizer=optimizer, model_parameters=model_parameters, training_data=training_data,
                 lr_scheduler=lr_scheduler, mpu=mpu, collate_fn=collate_fn, config=cfg)
    return engine, engine.optimizer, engine.training_dataloader, engine.lr_scheduler


__all__ = ['initialize', 'MSAMPDeepSpeedConfig', 'MSAMPDeepSpeedEngine', 'MSAMPPipelineEngine', 'PipelineModule']
