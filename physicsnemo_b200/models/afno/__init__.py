from .afno import AFNO
