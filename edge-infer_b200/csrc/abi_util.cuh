// Exception -> status mapping shared by the C-ABI translation units.
#pragma once

#include <new>
#include <stdexcept>
#include <string>

#include "common.cuh"

namespace ei {

extern thread_local std::string g_last_error;

struct PoisonedError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// Runs `body`; maps the reference API's exception classes to ei_status and records the message.
template <typename Body>
ei_status guarded(Body&& body) noexcept {
  try {
    body();
    return EI_OK;
  } catch (const PoisonedError& e) {
    g_last_error = e.what();
    return EI_POISONED;
  } catch (const std::length_error& e) {
    g_last_error = e.what();
    return EI_LENGTH;
  } catch (const std::out_of_range& e) {
    g_last_error = e.what();
    return EI_OUT_OF_RANGE;
  } catch (const std::invalid_argument& e) {
    g_last_error = e.what();
    return EI_INVALID_ARGUMENT;
  } catch (const std::overflow_error& e) {
    g_last_error = e.what();
    return EI_OVERFLOW;
  } catch (const std::logic_error& e) {
    g_last_error = e.what();
    return EI_LOGIC;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return EI_RUNTIME;
  } catch (...) {
    g_last_error = "unknown failure";
    return EI_RUNTIME;
  }
}

}  // namespace ei
