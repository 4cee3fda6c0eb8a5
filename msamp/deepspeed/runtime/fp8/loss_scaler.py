"""Static and dynamic loss scaling (the policy DeepSpeed's fp16 optimizers use)."""


class LossScaler:
    """Constant loss scale."""
    dynamic = False

    def __init__(self, scale=1.0):
        self.cur_scale = float(scale)

    @property
    def loss_scale(self):
        return self.cur_scale

    def update_scale(self, overflow):
        pass

    def state_dict(self):
        return {'cur_scale': self.cur_scale}

    def load_state_dict(self, sd):
        self.cur_scale = sd['cur_scale']


class DynamicLossScaler(LossScaler):
    """Halve on overflow (after ``hysteresis`` consecutive overflows), double after ``scale_window`` clean steps."""
    dynamic = True

    def __init__(self, init_scale=2**16, scale_factor=2.0, scale_window=1000, min_scale=1.0, hysteresis=2):
        super().__init__(init_scale)
        self.cur_iter = 0
        self.last_overflow_iter = -1
        self.scale_factor, self.scale_window, self.min_scale = scale_factor, scale_window, min_scale
        self.hysteresis, self.cur_hysteresis = hysteresis, hysteresis

    def update_scale(self, overflow):
        if overflow:
            if self.hysteresis == 1 or self.cur_hysteresis == 1:
                self.cur_scale = max(self.cur_scale / self.scale_factor, self.min_scale)
            else:
                self.cur_hysteresis -= 1
            self.last_overflow_iter = self.cur_iter
        else:
            if (self.cur_iter - self.last_overflow_iter) % self.scale_window == 0:
                self.cur_hysteresis = self.hysteresis
                self.cur_scale *= self.scale_factor
        self.cur_iter += 1

    def state_dict(self):
        return {k: getattr(self, k) for k in ('cur_scale', 'cur_iter', 'last_overflow_iter', 'scale_factor', 'scale_window', 'min_scale',
                                              'hysteresis', 'cur_hysteresis')}

    def load_state_dict(self, sd):
        for k, v in sd.items():
            setattr(self, k, v)
