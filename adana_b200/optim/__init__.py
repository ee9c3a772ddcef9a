"""Optimizers and learning-rate schedules."""
from .adam_family import AdamWDecayingWD, AdEMAMix, AdEMAMix_DecayingWD, AdEMAMixDecayingWD
from .logtime import DANA_STAR_MK4, ADana, DanaStarMK4, logtime_update_, wd_multiplier
from .muon import CombinedScheduler, DistributedMuon, Manau, Muon, newton_schulz5, zeropower_via_newtonschulz5
from .schedule import (build_scheduler, cos_inf_schedule, powerlaw_schedule_with_warmup, wsd_schedule)
