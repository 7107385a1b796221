// bonsai_oracle_model.h - block-level and whole-token CPU restatement (test infrastructure only).
#ifndef BONSAI_ORACLE_MODEL_H
#define BONSAI_ORACLE_MODEL_H
#include "bonsai_oracle.h"
#endif
